"""Unpad / pad glue for padded batches, computed on the device with no host read-back.

Mirrors `_get_unpad_data`, `index_first_axis`, `_upad_input` and `pad_input` of
src/turbot5/model/padding.py (:79-88, :46-76, :113-150, :30-44).  The reference
reads the longest length back to the host (`.item()`, padding.py:82); here the
packed buffers are sized for the worst case (B*L rows) and the kernels take the
lengths from the device, so a forward pass never synchronises.
"""
from typing import NamedTuple

import torch

from . import _native as nat


class UnpadPlan(NamedTuple):
    seqlens: torch.Tensor      # int32 (B,)
    cu_seqlens: torch.Tensor   # int32 (B+1,)
    dest: torch.Tensor         # int32 (B*L,): packed row of each kept token, negative for padding
    batch: int
    seqlen: int


def get_unpad_plan(attention_mask: torch.Tensor) -> UnpadPlan:
    """mask (B, L), non-zero = keep -> lengths, cumulative lengths, destination rows."""
    nat.require_cuda(attention_mask)
    if attention_mask.dim() != 2:
        raise ValueError("attention_mask must be (batch, seqlen)")
    if attention_mask.dtype == torch.bool:
        attention_mask = attention_mask.view(torch.uint8)
    if attention_mask.is_floating_point():
        attention_mask = attention_mask != 0
        attention_mask = attention_mask.view(torch.uint8)
    m = attention_mask.contiguous()
    B, L = m.shape
    dev = m.device
    seqlens = torch.empty(B, dtype=torch.int32, device=dev)
    cu = torch.empty(B + 1, dtype=torch.int32, device=dev)
    dest = torch.empty(B * L, dtype=torch.int32, device=dev)
    if B == 0:
        cu.zero_()
    with torch.cuda.device(dev):
        nat.check(nat.lib().t5b_unpad_plan(m.data_ptr(), m.element_size(), B, L, seqlens.data_ptr(),
                                           cu.data_ptr(), dest.data_ptr(), nat.stream_ptr(dev)), "get_unpad_plan")
    return UnpadPlan(seqlens, cu, dest, B, L)


def _rows(t: torch.Tensor, n_rows: int):
    t2 = t.reshape(n_rows, -1)
    if t2.stride(-1) != 1 or (t2.stride(0) * t2.element_size()) % 16 or t2.data_ptr() % 16:
        t2 = t2.contiguous()
    return t2


def unpad_rows(x: torch.Tensor, plan: UnpadPlan) -> torch.Tensor:
    """(B, L, ...) -> packed (B*L, ...): kept tokens first, in order; the unused tail is zero.
    Differentiable: the gradient is the scatter back (`pad_rows`)."""
    if torch.is_grad_enabled() and x.requires_grad:
        return _Unpad.apply(x, plan)
    return _unpad_rows(x, plan)


def pad_rows(packed: torch.Tensor, plan: UnpadPlan) -> torch.Tensor:
    """packed (>= total kept rows, ...) -> (B, L, ...) with zeros at padded positions.
    Differentiable: the gradient is the gather (`unpad_rows`)."""
    if torch.is_grad_enabled() and packed.requires_grad:
        return _Pad.apply(packed, plan)
    return _pad_rows(packed, plan)


class _Unpad(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, plan):
        ctx.plan = plan
        return _unpad_rows(x, plan)

    @staticmethod
    def backward(ctx, g):
        return _pad_rows(g, ctx.plan), None


class _Pad(torch.autograd.Function):
    @staticmethod
    def forward(ctx, packed, plan):
        ctx.plan, ctx.rows = plan, packed.shape[0]
        return _pad_rows(packed, plan)

    @staticmethod
    def backward(ctx, g):
        gp = _unpad_rows(g, ctx.plan)            # B*L rows, kept tokens first, zero tail
        if gp.shape[0] != ctx.rows:
            if gp.shape[0] > ctx.rows:
                gp = gp[: ctx.rows]
            else:
                gp = torch.cat([gp, gp.new_zeros((ctx.rows - gp.shape[0],) + tuple(gp.shape[1:]))])
        return gp, None


def _unpad_rows(x: torch.Tensor, plan: UnpadPlan) -> torch.Tensor:
    nat.require_cuda(x)
    n = plan.batch * plan.seqlen
    src = _rows(x, n)
    row_bytes = src.shape[1] * src.element_size()
    if row_bytes % 16:
        raise ValueError("row size must be a multiple of 16 bytes")
    out = torch.empty((n, src.shape[1]), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        nat.check(nat.lib().t5b_gather_rows(src.data_ptr(), src.stride(0) * src.element_size(), out.data_ptr(),
                                            row_bytes, plan.dest.data_ptr(), n, row_bytes,
                                            nat.stream_ptr(x.device)), "unpad_rows")
    return out.view(n, *x.shape[2:])


def _pad_rows(packed: torch.Tensor, plan: UnpadPlan) -> torch.Tensor:
    nat.require_cuda(packed)
    n = plan.batch * plan.seqlen
    src = _rows(packed, packed.shape[0])
    row_bytes = src.shape[1] * src.element_size()
    if row_bytes % 16:
        raise ValueError("row size must be a multiple of 16 bytes")
    out = torch.empty((n, src.shape[1]), dtype=packed.dtype, device=packed.device)
    with torch.cuda.device(packed.device):
        nat.check(nat.lib().t5b_scatter_rows(src.data_ptr(), src.stride(0) * src.element_size(), out.data_ptr(),
                                             row_bytes, plan.dest.data_ptr(), n, row_bytes,
                                             nat.stream_ptr(packed.device)), "pad_rows")
    return out.view(plan.batch, plan.seqlen, *packed.shape[1:])
