"""``attention_host``: ``attention`` for inputs that live in pinned host memory.

Attention is independent per KV head and the query heads that share it, so the host tensors are
processed one KV-head group at a time on three streams: while group ``i`` is being computed, the
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
                   device=None, out: torch.Tensor | None = None, kv_heads_per_chunk: int = 1) -> torch.Tensor:
    """q ``[B, Hq, Sq, D]``, k / v ``[B, Hkv, Skv, D]`` in (pinned) host memory -> host ``[B, Hq, Sq, D]``.

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
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    group = hq // hkv
    if out is None:
        out = torch.empty((b, hq, sq, d), dtype=q.dtype).pin_memory()
    elif out.is_cuda or tuple(out.shape) != (b, hq, sq, d) or out.dtype != q.dtype:
        raise ValueError("out must be a host tensor shaped and typed like q")

    compute = torch.cuda.current_stream(dev)
    copy_in, copy_out = _side_streams(dev)
    copy_in.wait_stream(compute)
    copy_out.wait_stream(compute)
    last_out = None
    staged = None
    chunks = [(h0, min(h0 + kv_heads_per_chunk, hkv)) for h0 in range(0, hkv, kv_heads_per_chunk)]

    def stage(h0, h1):
        with torch.cuda.stream(copy_in):
            parts = (q[:, h0 * group:h1 * group], k[:, h0:h1], v[:, h0:h1])
            on_dev = tuple(torch.empty(t.shape, dtype=t.dtype, device=dev).copy_(t, non_blocking=True) for t in parts)
            ready = torch.cuda.Event()
            ready.record(copy_in)
        return on_dev, ready

    staged = stage(*chunks[0])
    for idx, (h0, h1) in enumerate(chunks):
        (qd, kd, vd), ready = staged
        if idx + 1 < len(chunks):
            staged = stage(*chunks[idx + 1])              # next group's inputs cross PCIe during this group's kernels
        compute.wait_event(ready)
        for t in (qd, kd, vd):
            t.record_stream(compute)
        od = attention(qd, kd, vd, config=config)
        done = torch.cuda.Event()
        done.record(compute)
        od.record_stream(copy_out)
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(done)
            out[:, h0 * group:h1 * group].copy_(od, non_blocking=True)
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
