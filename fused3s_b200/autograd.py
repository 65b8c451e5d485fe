"""Differentiable fused sparse attention: ``torch.autograd`` around ``f3s_forward_lse`` and
``f3s_backward``.

The reference's extension has forward ops only (src/F3S.cpp:298-305) and its scripts run under
``torch.no_grad`` semantics; a graph-transformer layer that is to be trained needs dQ, dK and dV.
Both passes use TC-block plans that are built once per graph: the plan of the graph for the
forward pass and dQ, the plan of the transposed graph for dK and dV.

    plan = TrainingPlan(rowptr, colidx, num_nodes, device)          # once per graph
    out = attention(q, k, v, plan, scale_divisor=math.sqrt(d))      # q, k, v: fp16 [N, d] or [N, H, d]
    out.sum().backward()                                            # q.grad, k.grad, v.grad (fp16)
"""
from __future__ import annotations

import numpy as np
import torch

from . import cabi


class TrainingPlan:
    """TC-block arrays of a square graph and of its transpose, on one device."""

    def __init__(self, rowptr, colidx, num_nodes: int, device="cuda", block_w: int = 16, symmetric: bool = False):
        """``symmetric=True``: the caller guarantees that the adjacency pattern equals its transpose
        (undirected graphs, molecule batches); the transposed plan is then the plan itself and neither
        the transposition nor the second preprocessing runs."""
        self.num_nodes = int(num_nodes)
        self.device = torch.device(device)
        to_dev = lambda a: (torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)) if isinstance(a, np.ndarray)
                            else a.to(torch.int32)).to(self.device)
        rp, ci = to_dev(rowptr), to_dev(colidx)
        with torch.cuda.device(self.device):
            self.tcb = cabi.preprocess(ci, rp, self.num_nodes, block_w)
            if symmetric:
                self.tcb_t = self.tcb
            else:
                rp_t, ci_t = cabi.transpose_csr(rp, ci, self.num_nodes)
                self.tcb_t = cabi.preprocess(ci_t, rp_t, self.num_nodes, block_w)


class _FusedAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, plan: TrainingPlan, scale_divisor: float):
        out, lse = cabi.forward_lse(plan.tcb, plan.num_nodes, q, k, v, scale_divisor)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.plan = plan
        ctx.scale_divisor = float(scale_divisor)
        return out

    @staticmethod
    def backward(ctx, d_out):
        q, k, v, out, lse = ctx.saved_tensors
        plan = ctx.plan
        dq, dk, dv = cabi.backward(plan.tcb, plan.tcb_t, plan.num_nodes, q, k, v, out, lse, d_out, ctx.scale_divisor,
                                   grad_dtype=torch.float16)
        return dq, dk, dv, None, None


def attention(q, k, v, plan: TrainingPlan, scale_divisor: float = 1.0):
    """softmax(mask(Q K^T / scale_divisor)) V over the plan's graph; fp16 inputs, fp32 output,
    differentiable with respect to q, k and v."""
    if q.dtype != torch.float16 or k.dtype != torch.float16 or v.dtype != torch.float16:
        raise cabi.F3SError(cabi.ERR_INVALID_ARG, "q, k, v must be fp16")
    return _FusedAttention.apply(q, k, v, plan, scale_divisor)


class _ShardedFusedAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q_local, k_local, v_local, att, scale_divisor: float):
        out, ctx.saved = att.forward_save(q_local, k_local, v_local, scale_divisor)
        ctx.att = att
        return out

    @staticmethod
    def backward(ctx, d_out):
        dq, dk, dv = ctx.att.backward_from(ctx.saved, d_out, grad_dtype=torch.float16)
        ctx.saved = None
        return dq, dk, dv, None, None


def sharded_attention(q_local, k_local, v_local, att, scale_divisor: float = 1.0):
    """Differentiable attention over a graph whose rows are divided over the ranks: ``att`` is this
    rank's ``fused3s_b200.sharding.ShardedTrainingAttention``; inputs and gradients are the rank's own
    rows (fp16), the collectives run inside.  Every call keeps its own saved tensors, so one ``att`` may be
    shared by several layers or micro-batches."""
    return _ShardedFusedAttention.apply(q_local, k_local, v_local, att, scale_divisor)
