"""Streaming checkpoint writer around the encode stage (the on-disk side of hi2/checkpoint.py:
``to_tensors`` / ``from_tensors`` :142-157, ``_batches`` :234-247, ``write_checkpoints`` :320-505,
shard markers :487-497) and a device-side ``verify``.

What is kept of the reference: the tensor names of the format (``<base>.hi2_codes``, ``.hi2_code_off``,
``.hi2_blk_params``, ``.hi2_param_off``, ``.hi2_row_consts``, ``.hi2_row_nbits``, ``.hi2_row_block``,
``.hi2_had``, optional ``.hi2_col_scale``), tensors that are not quantised passed through under their
own names, consecutive tensors batched under a byte budget for the encode, a shard written to a
temporary file and renamed, and a JSON marker beside it carrying the file's SHA-256 and a short
report per tensor.  What is B200-specific: a batch is encoded with the packed buffers LEFT ON THE
DEVICE, copied to pinned host memory on a copy stream while the next batch is being encoded, and
only then handed to the safetensors writer (the reference assembles on the device but copies
synchronously, hi2/format.py:172-184).  With ``moe_layout="stacked"`` the routed experts of a layer
and projection group are written as one stack (hi2/stack.py, ``--moe-layout stacked``), assembled on
the device from the packed buffers of the shard before the copy to the host.  Reading source
shards, resuming, validation of foreign files and the dense / portable exports stay with the
reference's ``checkpoint.py``.
"""

from __future__ import annotations

import hashlib
import json
import os
from pathlib import Path

import torch

from .calibrate import Config, EncodeRequest, encode_many
from .format import FIELDS, HI2Tensor, dequantize
from .moe import expert_parts
from .stack import LAYOUTS, MARK, PART_GROUP, split_stack, stack_packed

ENCODE_BATCH_BYTES = int(float(os.environ.get("HI2_ENCODE_BATCH_GB", "6")) * 2**30)


def to_tensors(t: HI2Tensor, base: str) -> dict:
    """``{safetensors name: tensor}`` of one packed tensor under ``base`` (the Linear's name without
    ``.weight``)."""
    out = {f"{base}.hi2_{f}": getattr(t, f) for f in FIELDS}
    if t.col_scale is not None:
        out[f"{base}.hi2_col_scale"] = t.col_scale
    return out


def from_tensors(d: dict, base: str) -> HI2Tensor:
    g = {f: d[f"{base}.hi2_{f}"] for f in FIELDS}
    return HI2Tensor(**g, shape=(g["row_nbits"].numel(), g["had"].numel() * 16), col_scale=d.get(f"{base}.hi2_col_scale"))


def batches(names, tables, budget: int = ENCODE_BATCH_BYTES):
    """Consecutive tensors grouped so that factor (K^2) and working copies (3 R K) of a group stay
    under ``budget`` bytes of fp32 (hi2/checkpoint.py:234-247)."""
    cur, size = [], 0
    for name in names:
        r, k = tables[name].shape
        need = 4 * (k * k + 3 * r * k)
        if cur and size + need > budget:
            yield cur
            cur, size = [], 0
        cur.append(name)
        size += need
    if cur:
        yield cur


def file_digest(path: Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 22), b""):
            h.update(chunk)
    return h.hexdigest()


def _report(t: HI2Tensor, table) -> dict:
    r, k = t.shape
    nb = t.row_nbits.to(torch.float64)
    bl = t.row_block.to(torch.float64)
    bits = float((nb * k + 16 * k / bl).sum()) + 48 * r + (16 * k if t.col_scale is not None else 0)
    return {"shape": [r, k], "bpw": bits / (r * k), "frac_int4": float((t.row_nbits == 4).float().mean()),
            "frac_int8": float((t.row_nbits == 8).float().mean()), "rotated_groups": int(t.had.sum()),
            "groups": int(t.had.numel()), "n_tokens": int(table.n_tokens)}


class _HostCopy:
    """Packed buffers of one batch (and, in the stacked layout, the expert stacks of a shard) on their
    way to pinned host memory, on a copy stream beside the encode of the next batch."""

    def __init__(self, packed: dict, stream: torch.cuda.Stream, stacks: dict | None = None):
        self.done = torch.cuda.Event()
        self.host, self.stacks = {}, {}
        stream.wait_stream(torch.cuda.current_stream())

        def pinned(v):
            if v is None or not v.is_cuda:
                return v
            h = torch.empty(v.shape, dtype=v.dtype, pin_memory=True)
            h.copy_(v, non_blocking=True)
            v.record_stream(stream)
            return h

        with torch.cuda.stream(stream):
            for name, t in packed.items():
                self.host[name] = HI2Tensor(**{f: pinned(getattr(t, f)) for f in FIELDS}, shape=t.shape,
                                            col_scale=pinned(t.col_scale))
            for base, arrays in (stacks or {}).items():
                self.stacks[base] = {f: pinned(v) for f, v in arrays.items()}
            self.done.record(stream)

    def result(self) -> dict:
        self.done.synchronize()
        return self.host


def write_shard(path: Path, packed: dict, passthrough: dict | None = None, tables: dict | None = None,
                stacks: dict | None = None, reports: dict | None = None) -> dict:
    """One safetensors file with the packed tensors of ``packed`` (``{'<base>.weight': HI2Tensor}``, on
    the host), the expert stacks of ``stacks`` (``{stack base: arrays}``, :func:`hi2_b200.stack.build_stack`)
    and the tensors of ``passthrough`` as they are; written to ``<path>.tmp`` and renamed;
    ``<path>.done.json`` records the SHA-256 of the file, its tensor names and a report per tensor
    (``reports`` carries those of tensors that went into stacks).  Returns the marker."""
    from safetensors.torch import save_file

    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    out, reports = {}, dict(reports or {})
    for name, t in packed.items():
        base = name.removesuffix(".weight")
        out.update({k: v.contiguous() for k, v in to_tensors(t, base).items()})
        if tables is not None and name in tables:
            reports[name] = _report(t, tables[name])
    for base, arrays in (stacks or {}).items():
        out.update({f"{base}.hi2_{f}": v.cpu().contiguous() for f, v in arrays.items()})
    for name, v in (passthrough or {}).items():
        out[name] = v.detach().cpu().contiguous()
    tmp = path.with_name(path.name + ".tmp")
    save_file(out, str(tmp), metadata={"format": "pt", "hi2": "rdna_hint_flex"})
    os.replace(tmp, path)
    marker = {"schema_version": 1, "shard": path.name, "sha256": file_digest(path), "tensor_names": sorted(out),
              "tensors": reports}
    mpath = path.with_name(path.name + ".done.json")
    mtmp = mpath.with_name(mpath.name + ".tmp")
    mtmp.write_text(json.dumps(marker, indent=1))
    os.replace(mtmp, mpath)
    return marker


def write_checkpoints(shards: dict, tables: dict, picks: dict, sigma_of, cfg: Config, out_dir,
                      budget: int = ENCODE_BATCH_BYTES, log=print, factors: dict | None = None,
                      moe_layout: str = "per-expert") -> dict:
    """Encode and write a model shard by shard.

    ``shards``: ``{file name: {tensor name: tensor on the device}}`` in source order; tensors with a
    table are quantised with ``picks[name]``, the others are passed through.  ``sigma_of(name)`` returns
    ``(second moment sum or None, tokens, sigma_id, ColumnStats or None)`` for a tensor - what
    :class:`hi2_b200.layerwise.DeviceSink` holds; ``factors`` (optional) its ``factors``: inverse
    factors already started while tabulating, by ``sigma_id``.  ``moe_layout="stacked"`` writes the
    routed experts of every layer and projection group that is complete in a shard as one stack; the
    packed buffers of the shard then stay on the device until the shard is encoded (a few GB), the
    stacks are put together there and copied to the host once.  Returns ``{file name: marker}``."""
    if moe_layout not in LAYOUTS:
        raise ValueError(f"moe_layout must be one of {LAYOUTS} (got {moe_layout!r})")
    out_dir = Path(out_dir)
    copy_stream = torch.cuda.Stream()
    markers = {}
    for shard, tensors in shards.items():
        quant = [n for n in tensors if n in tables]
        pending: list[_HostCopy] = []
        on_device: dict = {}
        for group in batches(quant, tables, budget):
            reqs = []
            for n in group:
                sigma, tokens, sid, stats = sigma_of(n)
                reqs.append(EncodeRequest(tensors[n], stats, tables[n], picks[n], sigma=sigma, sigma_id=sid,
                                          sigma_n=max(int(tokens), 1)))
            packed = dict(zip(group, encode_many(reqs, cfg, to_host=False, factors=factors)))
            if moe_layout == "stacked":
                on_device.update(packed)
            else:
                pending.append(_HostCopy(packed, copy_stream))  # D2H runs beside the next group's encode
        reports = {}
        if on_device:
            stacks, rest = stack_packed(on_device)
            reports = {n: _report(t, tables[n]) for n, t in on_device.items() if n not in rest}
            pending.append(_HostCopy(rest, copy_stream, stacks))
            del on_device
        host, host_stacks = {}, {}
        for p in pending:
            host.update(p.result())
            host_stacks.update(p.stacks)
        markers[shard] = write_shard(out_dir / shard, host, {n: v for n, v in tensors.items() if n not in tables}, tables,
                                     host_stacks, reports)
        log(f"{shard}: {len(quant)} tensors encoded ({len(host_stacks)} expert stacks), "
            f"{len(tensors) - len(quant)} passed through")
    return markers


def verify_checkpoint(out_dir, shards: dict, tables: dict, rtol: float = 0.35, log=print) -> dict:
    """Read every written shard back, check the marker's digest and tensor coverage, rebuild each
    packed tensor (from its own arrays, or out of the expert stack that holds it), dequantise it on
    the device (:func:`hi2_b200.format.dequantize`) and compare it with the source weight:
    ``{tensor name: relative Frobenius error}``; raises on a digest or coverage mismatch or an error
    above ``rtol``."""
    from safetensors import safe_open

    out_dir = Path(out_dir)
    errors = {}
    for shard, tensors in shards.items():
        path = out_dir / shard
        marker = json.loads((path.with_name(path.name + ".done.json")).read_text())
        if marker.get("sha256") != file_digest(path):
            raise ValueError(f"{path}: digest differs from its marker")
        with safe_open(str(path), "pt") as f:
            keys = set(f.keys())
            if keys != set(marker["tensor_names"]):
                raise ValueError(f"{path}: tensor coverage differs from its marker")
            members: dict = {}  # stack base -> its pieces, split once

            def packed_tensor(base):
                if f"{base}.hi2_codes" in keys:
                    return from_tensors({k: f.get_tensor(k) for k in keys if k.startswith(base + ".hi2_")}, base)
                ep = expert_parts(base)
                if ep is None or ep[2] not in PART_GROUP:
                    raise ValueError(f"{path}: no packed tensor for {base}")
                group, part = PART_GROUP[ep[2]]
                stack = f"{ep[0]}.{group}"
                if f"{stack}.hi2_{MARK}" not in keys:
                    raise ValueError(f"{path}: no packed tensor and no stack for {base}")
                if stack not in members:
                    arrays = {k.rsplit(".hi2_", 1)[1]: f.get_tensor(k) for k in keys if k.startswith(stack + ".hi2_")}
                    nparts = sum(1 for p, (g, _) in PART_GROUP.items() if g == group)
                    members[stack] = split_stack(arrays, nparts)
                return members[stack][ep[1]][part]

            for name, w in tensors.items():
                if name not in tables:
                    if not torch.equal(f.get_tensor(name), w.detach().cpu()):
                        raise ValueError(f"{path}: {name} was not passed through unchanged")
                    continue
                rec = dequantize(packed_tensor(name.removesuffix(".weight")), w.device)
                err = float((rec - w.double()).norm() / w.double().norm().clamp_min(1e-30))
                errors[name] = err
                if not err <= rtol:
                    raise ValueError(f"{path}: {name} reconstructs with relative error {err:.3f}")
    log(f"verified {len(errors)} packed tensors")
    return errors


__all__ = ["to_tensors", "from_tensors", "batches", "write_shard", "write_checkpoints", "verify_checkpoint",
           "file_digest", "ENCODE_BATCH_BYTES"]
