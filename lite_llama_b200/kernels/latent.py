"""Latent attention pieces (csrc/latent_attention.cu, csrc/gemm_simt.cu): queries and keys / values go through
low-rank latents, the cache holds one row ``[latent | rotated key part]`` per token, and the queries are multiplied
into the latent space so that ``sink_attention`` runs on the cached rows directly.  The reference's attention caches
full per-head keys and values (lite_llama/models/base.py:76-79) and has no counterpart."""

from __future__ import annotations

import torch

from ._common import check, float_code, lib, ptr, require_cuda, stream_handle


@torch.no_grad()
def rope_table(positions: torch.Tensor, rot_dims: int, rot_base: float) -> torch.Tensor | None:
    """fp32 ``[T, rot_dims]`` = per token ``[cos | sin]`` of ``position * base^(-2i / rot_dims)`` (angles in fp64); one
    table per step serves every layer with these rotary constants.  ``None`` when nothing rotates."""
    require_cuda(positions)
    if rot_dims == 0:
        return None
    out = torch.empty((positions.numel(), rot_dims), dtype=torch.float32, device=positions.device)
    check(lib().b2l_rope_table(out.data_ptr(), positions.data_ptr(), positions.numel(), rot_dims, float(rot_base),
                               stream_handle()))
    return out


@torch.no_grad()
def latent_prepare(proj: torch.Tensor, pool: torch.Tensor, kv_rows: torch.Tensor, cos_sin: torch.Tensor | None,
                   q_norm: torch.Tensor, kv_norm: torch.Tensor, q_rank: int, kv_rank: int, rot_dim: int,
                   rot_dims: int, eps: float) -> None:
    """Per token of the fused down-projection ``proj [T, >= q_rank + kv_rank + rot_dim]``: RMS norm of the query latent
    in place, RMS norm of the key/value latent and the rotation (``rope_table`` rows) of the shared key part into pool
    row ``kv_rows[t]``."""
    require_cuda(proj, pool, kv_rows, cos_sin, q_norm, kv_norm)
    if proj.stride(-1) != 1 or pool.stride(-1) != 1 or pool.shape[1] < kv_rank + rot_dim:
        raise ValueError("latent_prepare: bad layout")
    check(lib().b2l_latent_prepare(proj.data_ptr(), proj.stride(0), pool.data_ptr(), pool.stride(0), kv_rows.data_ptr(),
                                   ptr(cos_sin), q_norm.data_ptr(), kv_norm.data_ptr(), proj.shape[0], q_rank,
                                   kv_rank, rot_dim, rot_dims, float(eps), float_code(proj, "proj"), stream_handle()))


@torch.no_grad()
def rope_heads(dst: torch.Tensor, dst_head_stride: int, src: torch.Tensor, src_head_stride: int,
               cos_sin: torch.Tensor | None, heads: int, width: int, rot_dims: int) -> None:
    """``dst[t, h, :width] = src[t, h, :width]`` with the first ``rot_dims`` entries rotated by the token's
    ``rope_table`` row (rotate-half pairing); ``dst`` / ``src`` are 2-D views whose rows hold the heads
    ``*_head_stride`` apart."""
    require_cuda(dst, src, cos_sin)
    check(lib().b2l_rope_heads(dst.data_ptr(), dst.stride(0), dst_head_stride, src.data_ptr(), src.stride(0),
                               src_head_stride, ptr(cos_sin), src.shape[0], heads, width, rot_dims,
                               float_code(src, "src"), stream_handle()))


@torch.no_grad()
def head_linear(out: torch.Tensor, out_head_stride: int, x: torch.Tensor, x_head_stride: int, w: torch.Tensor,
                gate: torch.Tensor | None = None) -> None:
    """``out[t, h, :n] = w[h] @ x[t, h, :k]`` for ``w [heads, n, k]``; optional ``gate [T, >= heads]``:
    ``out[t, h] *= sigmoid(gate[t, h])``.  fp32 sums in ascending k, any dtype of the layer-list models (16-bit aligned
    operands: ``mma.sync`` tiles, csrc/gemm_rows_mma.cu; fp32 or odd shapes: CUDA cores, csrc/gemm_simt.cu)."""
    require_cuda(out, x, w, gate)
    heads, n, k = w.shape
    if w.dtype != x.dtype or not w.is_contiguous() or x.stride(-1) != 1 or out.stride(-1) != 1:
        raise ValueError("head_linear: bad layout")
    L, code = lib(), float_code(x, "x")
    # 16-bit operands with 16-byte aligned rows run on the tensor cores, everything else on the CUDA cores
    fn = L.b2l_head_linear_mma if L.b2l_rows_gemm_mma_ok(x.data_ptr(), w.data_ptr(), k, x.stride(0), x_head_stride, code) \
        else L.b2l_head_linear
    check(fn(out.data_ptr(), out.stride(0), out_head_stride, x.data_ptr(), x.stride(0), x_head_stride, w.data_ptr(),
             ptr(gate), gate.stride(0) if gate is not None else 0, x.shape[0], heads, n, k, code, stream_handle()))
