"""Dense projection ``x @ w.T (+ bias)`` on tcgen05.

Stands in for the reference's ``F.linear`` call sites
(lite_llama/models/quantization/methods/unquantized.py:21-22, lite_llama/models/base.py:489).
"""

from __future__ import annotations

import torch

from ._common import check, counters, dtype_code, float_code, lib, ptr, require_cuda, stream_handle, workspace


@torch.no_grad()
def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``[..., K] @ [N, K].T -> [..., N]`` in ``x``'s dtype, fp32 accumulation."""
    require_cuda(x, weight, bias)
    if x.dtype == torch.float32 or x.shape[-1] % 8 != 0:
        return linear_simt(x, weight, bias)       # exact fp32, or a K the TMA tiles cannot start on
    code = dtype_code(x, "x")
    if weight.dtype != x.dtype:
        raise ValueError(f"weight dtype {weight.dtype} must match activation dtype {x.dtype}")
    n, k = weight.shape
    if x.shape[-1] != k:
        raise ValueError(f"x has {x.shape[-1]} cols but weight expects {k}")
    if weight.stride(-1) != 1:
        weight = weight.contiguous()
    leading = x.shape[:-1]
    a = x.reshape(-1, k)
    if a.stride(-1) != 1 or a.stride(0) % 8 != 0 or a.data_ptr() % 16 != 0:
        a = a.contiguous()
    m = a.shape[0]
    out = torch.empty((m, n), dtype=x.dtype, device=x.device)
    if bias is not None:
        bias = bias.to(x.dtype).contiguous()
    L = lib()
    nbytes = L.b2l_linear_workspace_bytes(m, n, k, 2)
    ws = workspace(nbytes, x.device)
    cnt = counters(x.device)
    check(
        L.b2l_linear(
            out.data_ptr(), a.data_ptr(), weight.data_ptr(), ptr(bias), m, n, k, a.stride(0), weight.stride(0),
            out.stride(0), ptr(ws), nbytes, cnt.data_ptr(), cnt.numel(), code, stream_handle(),
        )
    )
    return out.reshape(*leading, n)


@torch.no_grad()
def linear_simt(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """The same product on the CUDA cores: fp32 accumulation in ascending k, any shape, fp16 / bf16 / TRUE fp32
    (no reduced-precision tensor mode).  A row's result does not depend on the other rows of the batch."""
    require_cuda(x, weight, bias)
    code = float_code(x, "x")
    if weight.dtype != x.dtype:
        raise ValueError(f"weight dtype {weight.dtype} must match activation dtype {x.dtype}")
    n, k = weight.shape
    if x.shape[-1] != k:
        raise ValueError(f"x has {x.shape[-1]} cols but weight expects {k}")
    if weight.stride(-1) != 1:
        weight = weight.contiguous()
    leading = x.shape[:-1]
    a = x.reshape(-1, k)
    if a.stride(-1) != 1:
        a = a.contiguous()
    out = torch.empty((a.shape[0], n), dtype=x.dtype, device=x.device)
    if bias is not None:
        bias = bias.to(x.dtype).contiguous()
    check(lib().b2l_gemm_simt(out.data_ptr(), a.data_ptr(), weight.data_ptr(), ptr(bias), a.shape[0], n, k,
                              a.stride(0), weight.stride(0), out.stride(0), code, stream_handle()))
    return out.reshape(*leading, n)
