"""Generic tensor utilities on the kernel library (``csrc/scan.cu``): prefix sums, row gather /
scatter / scatter-add, pitched copies, 2-D transpose, 32-bit fill.  CPU tensors take the
equivalent PyTorch expression.  The reference lists ``scan``, ``gather``, ``scatter`` and
``memory`` kernel files in build.zig:149-161 and ships none of them."""
from __future__ import annotations

import torch

from . import _lib


def cumsum(x: torch.Tensor, exclusive: bool = False, reverse: bool = False) -> torch.Tensor:
    """Prefix sum along the last dimension of an fp32 tensor.  ``reverse`` sums from the end
    (suffix sums); ``exclusive`` leaves the element itself out."""
    if not x.is_cuda:
        xf = x.float().flip(-1) if reverse else x.float()
        y = xf.cumsum(-1)
        if exclusive:
            y = y - xf
        return y.flip(-1) if reverse else y
    assert x.dtype == torch.float32
    xc = x.contiguous()
    n = xc.shape[-1]
    rows = xc.numel() // max(n, 1)
    y = torch.empty_like(xc)
    if xc.numel() == 0:
        return y
    L = _lib.lib()
    need = L.ceo_cumsum_scratch_floats(rows, n)
    scratch = _lib.scratch(xc.device, need, "scan") if need else None
    _lib.check(L.ceo_cumsum_f32(xc.data_ptr(), y.data_ptr(), rows, n, int(exclusive), int(reverse),
                                _lib.ptr(scratch), _lib.stream()), "ceo_cumsum_f32")
    return y


def _row_bytes(t: torch.Tensor) -> int:
    rb = t[0].numel() * t.element_size() if t.shape[0] else 0
    if rb % 16:
        raise ValueError("rows must be a multiple of 16 bytes")
    return rb


def gather_rows(src: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """out[i] = src[idx[i]] over the first dimension; indices out of range give zero rows."""
    if not src.is_cuda:
        ok = (idx >= 0) & (idx < src.shape[0])
        out = src[idx.clamp(0, src.shape[0] - 1)]
        return out * ok.view(-1, *([1] * (src.dim() - 1))).to(out.dtype)
    src = src.contiguous()
    idx = idx.contiguous().long()
    out = torch.empty((idx.numel(),) + tuple(src.shape[1:]), dtype=src.dtype, device=src.device)
    if idx.numel():
        _lib.check(_lib.lib().ceo_gather_rows(idx.data_ptr(), src.data_ptr(), out.data_ptr(),
                                              idx.numel(), _row_bytes(src), src.shape[0],
                                              _lib.stream()), "ceo_gather_rows")
    return out


def scatter_rows(dst: torch.Tensor, idx: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """dst[idx[i]] = src[i] in place (indices out of range are skipped; for duplicate indices
    one writer wins)."""
    if not dst.is_cuda:
        ok = (idx >= 0) & (idx < dst.shape[0])
        dst[idx[ok]] = src[ok]
        return dst
    assert dst.is_contiguous() and dst.dtype == src.dtype and dst.shape[1:] == src.shape[1:]
    src = src.contiguous()
    idx = idx.contiguous().long()
    if idx.numel():
        _lib.check(_lib.lib().ceo_scatter_rows(idx.data_ptr(), src.data_ptr(), dst.data_ptr(),
                                               idx.numel(), _row_bytes(dst), dst.shape[0],
                                               _lib.stream()), "ceo_scatter_rows")
    return dst


def scatter_add_rows(dst: torch.Tensor, idx: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """dst[idx[i]] += src[i] in place, fp32 rows (duplicates accumulate)."""
    if not dst.is_cuda:
        ok = (idx >= 0) & (idx < dst.shape[0])
        return dst.index_add_(0, idx[ok], src[ok].to(dst.dtype))
    assert dst.is_contiguous() and dst.dtype == torch.float32 and src.dtype == torch.float32
    src = src.contiguous()
    idx = idx.contiguous().long()
    D = dst[0].numel()
    if idx.numel():
        _lib.check(_lib.lib().ceo_scatter_add_f32(idx.data_ptr(), src.data_ptr(), dst.data_ptr(),
                                                  idx.numel(), D, dst.shape[0], _lib.stream()),
                   "ceo_scatter_add_f32")
    return dst


def copy2d(dst: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """Copies a 2-D tensor whose rows are contiguous (any row pitch) into another such tensor."""
    assert dst.shape == src.shape and dst.dtype == src.dtype and dst.dim() == 2
    if not dst.is_cuda:
        return dst.copy_(src)
    assert dst.stride(1) == 1 and src.stride(1) == 1
    es = dst.element_size()
    _lib.check(_lib.lib().ceo_copy2d(src.data_ptr(), src.stride(0) * es, dst.data_ptr(),
                                     dst.stride(0) * es, dst.shape[0], dst.shape[1] * es,
                                     _lib.stream()), "ceo_copy2d")
    return dst


def transpose2d(x: torch.Tensor) -> torch.Tensor:
    """A contiguous transpose of a 2-D tensor of 2-byte elements (bf16 / fp16 / int16)."""
    assert x.dim() == 2
    if not x.is_cuda:
        return x.t().contiguous()
    assert x.element_size() == 2 and x.stride(1) == 1
    out = torch.empty(x.shape[1], x.shape[0], dtype=x.dtype, device=x.device)
    _lib.check(_lib.lib().ceo_transpose16(x.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1],
                                          x.stride(0), out.stride(0), _lib.stream()),
               "ceo_transpose16")
    return out


def memset32(x: torch.Tensor, value: int) -> torch.Tensor:
    """Fills a contiguous tensor of 4-byte elements with one 32-bit pattern."""
    assert x.is_contiguous() and x.element_size() == 4
    if not x.is_cuda:
        x.view(torch.int32).fill_(value if value < 2 ** 31 else value - 2 ** 32)
        return x
    v = value if value < 2 ** 31 else value - 2 ** 32
    _lib.check(_lib.lib().ceo_memset32(x.data_ptr(), x.numel(), v, _lib.stream()), "ceo_memset32")
    return x
