"""Multi-GPU plan of the encode path: one process per GPU, ``torch.distributed`` underneath.

The path shards in two ways and needs exactly two exchanges:

* tokens - every rank accumulates the second moment of ITS calibration tokens for every shared
  input; the partial sums (fp32 ``[K, K]``) are then reduced to the rank that owns the input
  (NCCL over NVLink; the reference adds per-device partials on its primary device,
  hi2/layerwise.py:221-229, hi2/hessian.py:42-44);
* matrices - tables, factorisation, GPTQ and packing of a matrix run entirely on its owner
  (hi2 shards rows and re-factorises on every device, hi2/calibrate.py:333-347, 399-405).
  The global allocation needs every table, so the ``sse`` tables (a few bytes per row) are
  all-gathered and each rank runs the same deterministic allocation.

Every function takes plain tensors so the logic is testable with ``gloo`` on CPU.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist


def init_from_env(device_type: str | None = None, timeout_s: float = 600.0):
    """Join the process group described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT.
    Returns ``(rank, world, device)``; a single process without those variables is rank 0 of 1."""
    import datetime

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if device_type is None:
        device_type = "cuda" if torch.cuda.is_available() else "cpu"
    device = torch.device(device_type, local) if device_type == "cuda" else torch.device("cpu")
    if device.type == "cuda":
        torch.cuda.set_device(device)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        kw = {"device_id": device} if device.type == "cuda" else {}
        dist.init_process_group(
            "nccl" if device.type == "cuda" else "gloo", rank=rank, world_size=world,
            timeout=datetime.timedelta(seconds=timeout_s), **kw,
        )
    return rank, world, device


def world_size() -> int:
    return dist.get_world_size() if dist.is_initialized() else 1


def rank() -> int:
    return dist.get_rank() if dist.is_initialized() else 0


def owner_of(index: int, world: int | None = None) -> int:
    """Round-robin owner of unit ``index`` (a layer, a shared input, an expert group)."""
    return index % (world or world_size())


def token_shard(tokens: int, r: int | None = None, world: int | None = None) -> tuple[int, int]:
    """Contiguous token range of rank ``r``: even split, remainder to the first ranks."""
    world = world or world_size()
    r = rank() if r is None else r
    base, extra = divmod(tokens, world)
    lo = r * base + min(r, extra)
    return lo, lo + base + (1 if r < extra else 0)


def reduce_second_moment(s: torch.Tensor, n: int, owner: int, async_op: bool = False,
                         n_total: int | None = None):
    """Sum partial second moments ``s`` (in place, fp32) onto ``owner`` and the token counts onto
    every rank.  Returns ``(n_total, work)``; ``work`` is None unless ``async_op``.  A caller that
    knows the total token count (the shards of :func:`token_shard` add up to it) passes ``n_total``
    and saves the count's all-reduce and the host synchronisation that reading it costs."""
    if world_size() == 1:
        return n, None
    if n_total is None:
        count = torch.tensor([n], dtype=torch.int64, device=s.device)
        dist.all_reduce(count)
        n_total = int(count.item())
    work = dist.reduce(s, dst=owner, op=dist.ReduceOp.SUM, async_op=async_op)
    return n_total, work


def reduce_scatter_second_moments(stack: torch.Tensor, async_op: bool = False):
    """``stack [world, K, K]`` (fp32): this rank's partial second moment of the same input of every
    unit, unit ``r`` owned by rank ``r``.  One reduce-scatter instead of ``world`` reductions onto
    single owners: every link carries ``(world - 1) / world`` of the stack once, and the switch can
    do the sums.  Returns ``(own [K, K] summed over the ranks, work)``."""
    if world_size() == 1:
        return stack[0], None
    if stack.shape[0] != world_size():
        raise ValueError("one slice per rank is needed")
    if dist.get_backend() == "gloo":  # gloo has no reduce-scatter: all-reduce and keep the own slice
        work = dist.all_reduce(stack, async_op=async_op)
        return stack[rank()], work
    out = torch.empty_like(stack[0])
    work = dist.reduce_scatter_tensor(out, stack, op=dist.ReduceOp.SUM, async_op=async_op)
    return out, work


def all_reduce_second_moment(s: torch.Tensor, n: int):
    """The all-reduce form (every rank ends with the full sum)."""
    if world_size() == 1:
        return n
    count = torch.tensor([n], dtype=torch.int64, device=s.device)
    dist.all_reduce(count)
    dist.all_reduce(s)
    return int(count.item())


def gather_tables(local: list) -> list:
    """Every rank's table summaries, in rank order then local order.  A summary is any picklable
    object holding CPU tensors (name, shape, candidates, energy, ``sse``)."""
    if world_size() == 1:
        return list(local)
    box: list = [None] * world_size()
    dist.all_gather_object(box, local)
    return [t for part in box for t in part]


def gather_error_tables(tables: list, make):
    """All ranks' error tables for the global allocation, rank order then local order.

    Only what the allocator reads crosses the wire: one small pickled record per table (name,
    shape, candidates, energy, token count, whether a smoothing vector is stored) and the ``sse``
    values themselves as ONE padded fp32 tensor per rank (``all_gather`` on the tables' device: NCCL
    for CUDA tensors, gloo for CPU ones).  ``make(**fields)`` builds a table object; local tables
    are returned as they are."""
    if world_size() == 1:
        return list(tables)
    meta = [dict(name=t.name, shape=tuple(t.shape), candidates=list(t.candidates), energy=float(t.energy),
                 n_tokens=t.n_tokens, scaled=t.col_scale is not None) for t in tables]
    box: list = [None] * world_size()
    dist.all_gather_object(box, meta)
    cmax = max(len(m["candidates"]) for part in box for m in part)
    rmax = max(sum(m["shape"][0] for m in part) for part in box)
    dev = tables[0].sse.device if tables else torch.device("cpu")
    mine = torch.full((cmax, rmax), float("inf"), dtype=torch.float32, device=dev)
    off = 0
    for t in tables:
        mine[: t.sse.shape[0], off : off + t.sse.shape[1]] = t.sse
        off += t.sse.shape[1]
    parts = [torch.empty_like(mine) for _ in range(world_size())]
    dist.all_gather(parts, mine)
    out = []
    for r, (part, buf) in enumerate(zip(box, parts)):
        if r == rank():
            out.extend(tables)
            continue
        off = 0
        for m in part:
            rows, c = m["shape"][0], len(m["candidates"])
            out.append(make(name=m["name"], shape=m["shape"], had=None, sse=buf[:c, off : off + rows],
                            candidates=m["candidates"], energy=m["energy"], n_tokens=m["n_tokens"],
                            col_scale=torch.empty(0) if m["scaled"] else None))
            off += rows
    return out


def gather_tables_known_layout(local: list, specs: list, make) -> list:
    """All error tables of a job whose table list every rank can write down beforehand.

    ``specs`` lists every table of the job in one global order as ``(owner rank, name, shape,
    candidates, n_tokens, has smoothing vector)``; ``local`` holds this rank's tables in that
    order.  Nothing but numbers crosses the wire and the host never waits: each rank sends ONE flat
    fp32 tensor (per table its energy, then ``sse [C, R]`` row-major; padded to the longest rank)
    through one ``all_gather``.  Returns table objects in the order of ``specs``; local ones are
    returned as they are, the others are built by ``make(**fields)`` around views of the gathered
    buffer."""
    if world_size() == 1:
        return list(local)
    me = rank()
    sizes = [0] * world_size()
    for owner, _, shape, cands, _, _ in specs:
        sizes[owner] += 1 + len(cands) * shape[0]
    if local:
        dev = local[0].sse.device
    else:
        dev = torch.device("cpu") if dist.get_backend() == "gloo" else torch.device("cuda", torch.cuda.current_device())
    mine = torch.zeros(max(sizes), dtype=torch.float32, device=dev)
    off = 0
    for t in local:
        e = t.energy if isinstance(t.energy, torch.Tensor) else torch.tensor(float(t.energy))
        n = t.sse.numel()
        mine[off] = e.to(dev, torch.float32).reshape(())
        mine[off + 1 : off + 1 + n] = t.sse.reshape(-1)
        off += 1 + n
    if off != sizes[me]:
        raise ValueError("local tables do not match the layout")
    parts = [torch.empty_like(mine) for _ in range(world_size())]
    dist.all_gather(parts, mine)
    offs = [0] * world_size()
    it = iter(local)
    out = []
    for owner, name, shape, cands, n_tokens, scaled in specs:
        if owner == me:
            out.append(next(it))
            continue
        buf, o = parts[owner], offs[owner]
        c, rows = len(cands), shape[0]
        out.append(make(name=name, shape=tuple(shape), had=None, sse=buf[o + 1 : o + 1 + c * rows].view(c, rows),
                        candidates=list(cands), energy=buf[o], n_tokens=n_tokens,
                        col_scale=torch.empty(0) if scaled else None))
        offs[owner] = o + 1 + c * rows
    return out


def barrier() -> None:
    if world_size() > 1:
        dist.barrier()
