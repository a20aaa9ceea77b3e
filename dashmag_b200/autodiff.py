"""The attention operator under automatic differentiation.

Mirrors crates/dash-ops/src/attention.rs:357-542: the ONE node Burn's ``Autodiff`` records for the
forward - its state is exactly ``(query, key, value, output, lse, mask, options)`` and its backward
is the library's written-out backward pass, nothing is re-traced - and the routing of the decoding
step when some input is tracked.  torch's autograd plays the part Burn's plays for the reference;
every computation is still a call through the C ABI (``dashmag_b200.attention``).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import attention as A
from .contract import AttentionMask, AttentionOptions


class AttentionNode(torch.autograd.Function):
    """crates/dash-ops/src/attention.rs:377-414 (``AttentionNode``, ``NodeState``) and :418-456
    (``autodiff_forward``).  Returns the output and the log-sum-exp; only the output carries a
    gradient (the reference hands the log-sum-exp back as an inner, untracked tensor)."""

    @staticmethod
    def forward(ctx, query, key, value, mask: AttentionMask, options: AttentionOptions):
        output, lse = A.attention_with_lse(query, key, value, mask, options)
        # What the backward pass needs: the inputs, the forward's output and log-sum-exp (saved
        # tensors), the mask and the options (plain data; the mask's tensors carry no gradient).
        ctx.save_for_backward(query, key, value, output, lse)
        ctx.mask, ctx.options = mask, options
        ctx.mark_non_differentiable(lse)
        return output, lse

    @staticmethod
    def backward(ctx, grad_output, _grad_lse):
        query, key, value, output, lse = ctx.saved_tensors
        if grad_output.stride(-1) != 1:
            grad_output = grad_output.contiguous()
        grad_query, grad_key, grad_value = A.attention_backward(query, key, value, output, lse, grad_output, ctx.mask, ctx.options)
        need = ctx.needs_input_grad
        return (grad_query if need[0] else None, grad_key if need[1] else None, grad_value if need[2] else None, None, None)


def _tracked(*tensors) -> bool:
    return torch.is_grad_enabled() and any(t.requires_grad for t in tensors)


def attention_with_lse(query, key, value, mask: AttentionMask = AttentionMask.none(),
                       options: AttentionOptions = AttentionOptions()):
    """``attention_with_lse`` for tensors that may be tracked: one node when any is, the plain call
    otherwise (``OpsKind::UnTracked``, :447-450)."""
    if _tracked(query, key, value):
        return AttentionNode.apply(query, key, value, mask, options)
    return A.attention_with_lse(query, key, value, mask, options)


def attention(query, key, value, mask: AttentionMask = AttentionMask.none(), options: AttentionOptions = AttentionOptions()):
    return attention_with_lse(query, key, value, mask, options)[0]


def reference_decode(query, key, value, cache_lengths, options: AttentionOptions):
    """The decoding step written in tensor operations that autograd records: what the reference
    falls back to for a TRACKED step with per-sequence lengths, which has no training path
    (crates/dash-ops/src/attention.rs:516-517, reference.rs:431-467).  f32 arithmetic; a sequence
    that holds no key gives zeros."""
    b, hq, d = query.shape
    s, hkv = key.shape[1], key.shape[2]
    group = hq // hkv
    scale = options.scale_for(d)
    q32 = query.float().view(b, hkv, group, d)
    scores = torch.einsum("bhgd,bshd->bhgs", q32, key.float()) * scale
    positions = torch.arange(s, device=query.device)
    lengths = (torch.full((b,), s, device=query.device) if cache_lengths is None
               else cache_lengths.to(torch.int64).clamp(0, s))
    visible = positions[None, :] < lengths[:, None]
    if options.window is not None and options.window.left is not None:
        visible &= positions[None, :] >= (lengths[:, None] - 1 - int(options.window.left))
    scores = scores.masked_fill(~visible[:, None, None, :], float("-inf"))
    top = scores.amax(dim=-1, keepdim=True)
    top = torch.where(torch.isfinite(top), top, torch.zeros_like(top))
    weights = torch.exp(scores - top)
    total = weights.sum(dim=-1, keepdim=True)
    weights = torch.where(total > 0, weights / total.clamp_min(1e-38), torch.zeros_like(weights))
    out = torch.einsum("bhgs,bshd->bhgd", weights, value.float())
    return out.reshape(b, hq, d).to(query.dtype)


def attention_decode(query, key, value, cache_lengths: Optional[torch.Tensor] = None,
                     options: AttentionOptions = AttentionOptions()):
    """The decoding step for tensors that may be tracked (crates/dash-ops/src/attention.rs:498-542):

    - nothing tracked: the decoding kernels;
    - tracked, every sequence holding all ``S`` keys: the TRAINING forward with one query, which sits
      after every key, so that its node's backward applies; causality changes nothing for it, and
      the reshapes around it carry the query's gradient back to ``[B, Hq, D]``;
    - tracked with per-sequence lengths: no training path exists - the reference in recorded tensor
      operations."""
    if not _tracked(query, key, value):
        return A.attention_decode(query, key, value, cache_lengths, options)
    if cache_lengths is None:
        b, hq, d = query.shape
        output = AttentionNode.apply(query.reshape(b, 1, hq, d), key, value, AttentionMask.none(), options.with_causal(False))[0]
        return output.reshape(b, hq, d)
    return reference_decode(query, key, value, cache_lengths, options)
