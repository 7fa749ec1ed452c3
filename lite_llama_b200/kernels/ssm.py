"""State-space mixer ops over ragged steps (csrc/ssm_scan.cu).  No reference counterpart."""

from __future__ import annotations

import torch

from ._common import check, float_code, lib, ptr, require_cuda, stream_handle


@torch.no_grad()
def causal_conv_silu(proj: torch.Tensor, col: int, channels: int, weight: torch.Tensor, bias: torch.Tensor,
                     tail: torch.Tensor, seq_start: torch.Tensor, seq_ctx: torch.Tensor, seq_slot: torch.Tensor):
    """``silu(conv(proj[:, col:col+channels]))`` per channel over a ragged step; ``tail [slots, taps-1, channels]``
    supplies the inputs of earlier steps and is advanced in place."""
    require_cuda(proj, weight, bias, tail, seq_start, seq_ctx, seq_slot)
    tokens = proj.shape[0]
    taps = weight.shape[1]
    out = torch.empty((tokens, channels), dtype=proj.dtype, device=proj.device)
    view = proj[:, col:col + channels]
    check(lib().b2l_causal_conv_silu(out.data_ptr(), view.data_ptr(), proj.stride(0), weight.data_ptr(), bias.data_ptr(),
                                     ptr(tail), seq_start.data_ptr(), seq_ctx.data_ptr(), seq_slot.data_ptr(),
                                     seq_ctx.numel(), tokens, channels, taps, float_code(proj, "proj"), stream_handle()))
    return out


@torch.no_grad()
def ssm_scan(xbc: torch.Tensor, dt_raw: torch.Tensor, dt_bias, a_log, d_skip, state: torch.Tensor,
             seq_start, seq_ctx, seq_slot, heads: int, groups: int, state_size: int, head_dim: int) -> torch.Tensor:
    """``y [tokens, heads*head_dim]`` fp32; ``state [slots, heads, state_size, head_dim]`` fp32 advanced in place.
    ``dt_raw`` is a column view ``[tokens, heads]`` of the input projection (row stride kept)."""
    require_cuda(xbc, dt_raw, state)
    if state.dtype != torch.float32:
        raise ValueError("ssm_scan: the recurrent state is fp32")
    tokens = xbc.shape[0]
    y = torch.empty((tokens, heads * head_dim), dtype=torch.float32, device=xbc.device)
    check(lib().b2l_ssm_scan(y.data_ptr(), state.data_ptr(), xbc.data_ptr(), xbc.stride(0), dt_raw.data_ptr(),
                             dt_raw.stride(0), dt_bias.data_ptr(), a_log.data_ptr(), d_skip.data_ptr(),
                             seq_start.data_ptr(), seq_ctx.data_ptr(), seq_slot.data_ptr(), seq_ctx.numel(), heads,
                             groups, state_size, head_dim, float_code(xbc, "xbc"), stream_handle()))
    return y


@torch.no_grad()
def gated_group_norm(y: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """``unit_rms(y * silu(z)) * weight`` with the statistic taken in ``groups`` equal parts; ``y`` fp32, ``z`` a
    column view of the projection, output in ``weight``'s dtype."""
    require_cuda(y, z, weight)
    rows, inner = y.shape
    out = torch.empty((rows, inner), dtype=weight.dtype, device=y.device)
    check(lib().b2l_gated_group_norm(out.data_ptr(), y.data_ptr(), z.data_ptr(), z.stride(0), weight.data_ptr(), rows,
                                     inner, groups, float(eps), float_code(weight, "weight"), stream_handle()))
    return out
