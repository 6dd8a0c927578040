"""``attention_host``: ``attention`` for inputs that live in pinned host memory.

Attention is independent per KV head and the query heads that share it, so the host tensors are
processed one KV-head group (or a few of its query heads) at a time on three streams: while group ``i`` is being computed, the
inputs of group ``i + 1`` cross PCIe and the result of group ``i - 1`` goes back.  Only two
groups' inputs and outputs are resident on the device at a time, which also bounds the device
memory of a long prompt to a fraction of the whole problem.  The reference has no host-side
entry point (its ``attention`` requires CUDA tensors, src/thriftattention/_checks.py:6-8); the
per-group results are exactly those of ``attention`` on the same slices.
"""
from __future__ import annotations

import torch

from .config import AttentionConfig
from .functional import attention


def attention_host(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, config: AttentionConfig | None = None,
                   device=None, out: torch.Tensor | None = None, kv_heads_per_chunk: int = 1,
                   q_heads_per_chunk: int = 0) -> torch.Tensor:
    """q ``[B, Hq, Sq, D]``, k / v ``[B, Hkv, Skv, D]`` in (pinned) host memory -> host ``[B, Hq, Sq, D]``.

    A chunk is ``kv_heads_per_chunk`` KV heads with all their query heads; with ``q_heads_per_chunk`` > 0 (it must
    divide the group size, and needs ``kv_heads_per_chunk == 1``) a KV head's query heads are processed that many at
    a time against K/V staged once — so that copies and kernels still overlap when a caller owns a single KV head.
    The call returns once every chunk has been queued; the result is complete after the current stream of
    ``device`` has been synchronised (``out`` is written by asynchronous copies, so it should be pinned too).
    """
    if q.is_cuda or k.is_cuda or v.is_cuda:
        raise ValueError("attention_host takes host tensors; call attention() for CUDA tensors")
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4 or k.shape != v.shape:
        raise ValueError("attention_host expects q [B,Hq,Sq,D] and k, v [B,Hkv,Skv,D]")
    b, hq, sq, d = q.shape
    hkv = k.shape[1]
    if hq % hkv != 0:
        raise ValueError("the number of query heads must be a multiple of the number of KV heads")
    if kv_heads_per_chunk < 1:
        raise ValueError("kv_heads_per_chunk must be positive")
    group = hq // hkv
    if q_heads_per_chunk and (kv_heads_per_chunk != 1 or q_heads_per_chunk < 0 or group % q_heads_per_chunk):
        raise ValueError("q_heads_per_chunk must divide the query heads per KV head and needs kv_heads_per_chunk == 1")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if out is None:
        out = torch.empty((b, hq, sq, d), dtype=q.dtype).pin_memory()
    elif out.is_cuda or tuple(out.shape) != (b, hq, sq, d) or out.dtype != q.dtype:
        raise ValueError("out must be a host tensor shaped and typed like q")

    compute = torch.cuda.current_stream(dev)
    copy_in, copy_out = _side_streams(dev)
    copy_in.wait_stream(compute)
    copy_out.wait_stream(compute)
    # work units: (first KV head, last KV head, first query head, last query head)
    units = []
    for h0 in range(0, hkv, kv_heads_per_chunk):
        h1 = min(h0 + kv_heads_per_chunk, hkv)
        step = q_heads_per_chunk or (h1 - h0) * group
        units += [(h0, h1, a, min(a + step, h1 * group)) for a in range(h0 * group, h1 * group, step)]

    def to_device(t):
        return torch.empty(t.shape, dtype=t.dtype, device=dev).copy_(t, non_blocking=True)

    def stage(unit, kv_cached):
        """Queue the unit's inputs on the copy stream; K/V are reused while the KV heads stay the same."""
        h0, h1, a, e = unit
        with torch.cuda.stream(copy_in):
            if kv_cached is not None and kv_cached[0] == (h0, h1):
                kd, vd = kv_cached[1], kv_cached[2]
            else:
                kd, vd = to_device(k[:, h0:h1]), to_device(v[:, h0:h1])
            qd = to_device(q[:, a:e])
            ready = torch.cuda.Event()
            ready.record(copy_in)
        return (qd, kd, vd, ready), ((h0, h1), kd, vd)

    last_out = None
    staged, kv_cached = stage(units[0], None)
    for idx, unit in enumerate(units):
        qd, kd, vd, ready = staged
        if idx + 1 < len(units):
            staged, kv_cached = stage(units[idx + 1], kv_cached)   # the next unit's inputs cross PCIe during this one's kernels
        compute.wait_event(ready)
        for t in (qd, kd, vd):
            t.record_stream(compute)
        od = attention(qd, kd, vd, config=config)
        done = torch.cuda.Event()
        done.record(compute)
        od.record_stream(copy_out)
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(done)
            out[:, unit[2]:unit[3]].copy_(od, non_blocking=True)
            last_out = torch.cuda.Event()
            last_out.record(copy_out)
    if last_out is not None:
        compute.wait_event(last_out)
    return out


_STREAMS: dict = {}


def _side_streams(dev: torch.device):
    key = (dev.type, dev.index)
    if key not in _STREAMS:
        _STREAMS[key] = (torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev))
    return _STREAMS[key]
