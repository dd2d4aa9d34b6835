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
synchronously, hi2/format.py:172-184).  Reading source shards, resuming, validation of foreign
files and the dense / portable exports stay with the reference's ``checkpoint.py``.
"""

from __future__ import annotations

import hashlib
import json
import os
from pathlib import Path

import torch

from .calibrate import Config, EncodeRequest, encode_many
from .format import FIELDS, HI2Tensor, dequantize

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
    """Packed buffers of one batch on their way to pinned host memory (a copy stream beside the
    encode of the next batch)."""

    def __init__(self, packed: dict, stream: torch.cuda.Stream):
        self.done = torch.cuda.Event()
        self.host = {}
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for name, t in packed.items():
                fields = {}
                for f in FIELDS:
                    v = getattr(t, f)
                    if v.is_cuda:
                        h = torch.empty(v.shape, dtype=v.dtype, pin_memory=True)
                        h.copy_(v, non_blocking=True)
                        v.record_stream(stream)
                        v = h
                    fields[f] = v
                cs = t.col_scale
                if cs is not None and cs.is_cuda:
                    h = torch.empty(cs.shape, dtype=cs.dtype, pin_memory=True)
                    h.copy_(cs, non_blocking=True)
                    cs.record_stream(stream)
                    cs = h
                self.host[name] = HI2Tensor(**fields, shape=t.shape, col_scale=cs)
            self.done.record(stream)

    def result(self) -> dict:
        self.done.synchronize()
        return self.host


def write_shard(path: Path, packed: dict, passthrough: dict | None = None, tables: dict | None = None) -> dict:
    """One safetensors file with the packed tensors of ``packed`` (``{'<base>.weight': HI2Tensor}``, on
    the host) and the tensors of ``passthrough`` as they are; written to ``<path>.tmp`` and renamed;
    ``<path>.done.json`` records the SHA-256 of the file, its tensor names and a report per tensor.
    Returns the marker."""
    from safetensors.torch import save_file

    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    out, reports = {}, {}
    for name, t in packed.items():
        base = name.removesuffix(".weight")
        out.update({k: v.contiguous() for k, v in to_tensors(t, base).items()})
        if tables is not None and name in tables:
            reports[name] = _report(t, tables[name])
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
                      budget: int = ENCODE_BATCH_BYTES, log=print, factors: dict | None = None) -> dict:
    """Encode and write a model shard by shard.

    ``shards``: ``{file name: {tensor name: tensor on the device}}`` in source order; tensors with a
    table are quantised with ``picks[name]``, the others are passed through.  ``sigma_of(name)`` returns
    ``(second moment sum or None, tokens, sigma_id, ColumnStats or None)`` for a tensor - what
    :class:`hi2_b200.layerwise.DeviceSink` holds; ``factors`` (optional) its ``factors``: inverse
    factors already started while tabulating, by ``sigma_id``.  Returns ``{file name: marker}``."""
    out_dir = Path(out_dir)
    copy_stream = torch.cuda.Stream()
    markers = {}
    for shard, tensors in shards.items():
        quant = [n for n in tensors if n in tables]
        pending: list[_HostCopy] = []
        for group in batches(quant, tables, budget):
            reqs = []
            for n in group:
                sigma, tokens, sid, stats = sigma_of(n)
                reqs.append(EncodeRequest(tensors[n], stats, tables[n], picks[n], sigma=sigma, sigma_id=sid,
                                          sigma_n=max(int(tokens), 1)))
            packed = dict(zip(group, encode_many(reqs, cfg, to_host=False, factors=factors)))
            pending.append(_HostCopy(packed, copy_stream))  # D2H runs beside the next group's encode
        host: dict = {}
        for p in pending:
            host.update(p.result())
        markers[shard] = write_shard(out_dir / shard, host, {n: v for n, v in tensors.items() if n not in tables}, tables)
        log(f"{shard}: {len(quant)} tensors encoded, {len(tensors) - len(quant)} passed through")
    return markers


def verify_checkpoint(out_dir, shards: dict, tables: dict, rtol: float = 0.35, log=print) -> dict:
    """Read every written shard back, check the marker's digest and tensor coverage, rebuild each
    packed tensor, dequantise it on the device (:func:`hi2_b200.format.dequantize`) and compare it
    with the source weight: ``{tensor name: relative Frobenius error}``; raises on a digest or
    coverage mismatch or an error above ``rtol``."""
    from safetensors import safe_open

    out_dir = Path(out_dir)
    errors = {}
    for shard, tensors in shards.items():
        path = out_dir / shard
        marker = json.loads((path.with_name(path.name + ".done.json")).read_text())
        if marker.get("sha256") != file_digest(path):
            raise ValueError(f"{path}: digest differs from its marker")
        with safe_open(str(path), "pt") as f:
            if set(f.keys()) != set(marker["tensor_names"]):
                raise ValueError(f"{path}: tensor coverage differs from its marker")
            for name, w in tensors.items():
                if name not in tables:
                    if not torch.equal(f.get_tensor(name), w.detach().cpu()):
                        raise ValueError(f"{path}: {name} was not passed through unchanged")
                    continue
                base = name.removesuffix(".weight")
                d = {k: f.get_tensor(k) for k in f.keys() if k.startswith(base + ".hi2_")}  # noqa: SIM118
                rec = dequantize(from_tensors(d, base), w.device)
                err = float((rec - w.double()).norm() / w.double().norm().clamp_min(1e-30))
                errors[name] = err
                if not err <= rtol:
                    raise ValueError(f"{path}: {name} reconstructs with relative error {err:.3f}")
    log(f"verified {len(errors)} packed tensors")
    return errors


__all__ = ["to_tensors", "from_tensors", "batches", "write_shard", "write_checkpoints", "verify_checkpoint",
           "file_digest", "ENCODE_BATCH_BYTES"]
