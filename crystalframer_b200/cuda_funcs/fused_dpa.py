"""autograd Function for the ragged softmax attention with logit and value biases."""
import torch

from .. import _lib
from .common import csr_offsets, f32c


class FusedDotProductAttentionCUDA(torch.autograd.Function):
    """Drop-in for models/cuda_funcs/fused_dpa.py:17-168.  ``que_ihk`` arrives already divided by
    sqrt(head_dim).  The backward pass recomputes probabilities from the saved log-sum-exp, so no
    (E,H) probability tensor and no transposed copies are kept."""

    @staticmethod
    def forward(ctx, que_ihk, key_ihk, val_ihk, aij_eh, bij_ehk, batch_i, edge_ij_e):
        N, H, K = que_ihk.shape
        E = edge_ij_e.shape[1]
        dev = que_ihk.device
        q, k, v = f32c(que_ihk), f32c(key_ihk), f32c(val_ihk)
        a, b = f32c(aij_eh), f32c(bij_ehk)
        edges = edge_ij_e.contiguous()
        e_start = csr_offsets(edges, N)
        out = torch.empty_like(v)
        lse = torch.empty((N, H), device=dev, dtype=torch.float32)
        p, ip = _lib.ptr, _lib.iptr
        _lib.invoke("cfb200_dpa_fwd", 1, dev, p(q), p(k), p(v), p(a), p(b), ip(edges), ip(e_start), N, E,
                    p(out), p(lse), None)
        ctx.save_for_backward(q, k, v, a, b, edges, e_start, out, lse)
        return out

    @staticmethod
    def backward(ctx, go_ihk):
        q, k, v, a, b, edges, e_start, out, lse = ctx.saved_tensors
        N, H, K = q.shape
        E = edges.shape[1]
        dev = q.device
        go = f32c(go_ihk)
        gq, gk, gv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        gz = torch.empty((E, H), device=dev, dtype=torch.float32)
        gb = torch.empty_like(b) if b is not None else None
        p, ip = _lib.ptr, _lib.iptr
        _lib.invoke("cfb200_dpa_bwd", 2, dev, p(q), p(k), p(v), p(a), p(b), ip(edges), ip(e_start), N, E,
                    p(out), p(lse), p(go), p(gq), p(gk), p(gv), p(gz), p(gb))
        return gq, gk, gv, (gz if a is not None else None), gb, None, None


def attention_probabilities(que_ihk, key_ihk, val_ihk, aij_eh, bij_ehk, edge_ij_e):
    """Forward pass that also returns the (E,H) probabilities (the reference keeps them as
    ``prob_eh``; used by tests and by callers that want attention weights)."""
    N, H, K = que_ihk.shape
    E = edge_ij_e.shape[1]
    dev = que_ihk.device
    q, k, v, a, b = f32c(que_ihk), f32c(key_ihk), f32c(val_ihk), f32c(aij_eh), f32c(bij_ehk)
    edges = edge_ij_e.contiguous()
    e_start = csr_offsets(edges, N)
    out = torch.empty_like(v)
    lse = torch.empty((N, H), device=dev, dtype=torch.float32)
    prob = torch.empty((E, H), device=dev, dtype=torch.float32)
    p, ip = _lib.ptr, _lib.iptr
    _lib.invoke("cfb200_dpa_fwd", 1, dev, p(q), p(k), p(v), p(a), p(b), ip(edges), ip(e_start), N, E,
                p(out), p(lse), p(prob))
    return out, prob, lse


class FusedDotProductAttentionSigmaMatCUDA(torch.autograd.Function):
    """Drop-in for models/cuda_funcs/fused_dpa_sigmamat.py:19-78: ragged softmax attention whose values are the
    six second-moment entries, output (N,H,6), no gradients.  ``que_ihk`` arrives divided by sqrt(head_dim);
    ``val_ihk`` (N,H,6) is added to the per-pair values ``bij_ehk`` (E,H,6) as in the reference.  Runs the
    attention kernel of FusedDotProductAttentionCUDA on the values padded to the head dimension."""

    @staticmethod
    def forward(ctx, que_ihk, key_ihk, val_ihk, aij_eh, bij_ehk, batch_i, edge_ij_e):
        N, H, K = que_ihk.shape
        E = edge_ij_e.shape[1]
        dev = que_ihk.device
        C = val_ihk.shape[-1]
        if C > K:
            raise RuntimeError("value width above the head dimension is not supported")
        q, k, a = f32c(que_ihk), f32c(key_ihk), f32c(aij_eh)
        v = torch.zeros((N, H, K), device=dev, dtype=torch.float32)
        v[..., :C] = val_ihk
        b = None
        if bij_ehk is not None:
            b = torch.zeros((E, H, K), device=dev, dtype=torch.float32)
            b[..., :C] = bij_ehk
        edges = edge_ij_e.contiguous()
        e_start = csr_offsets(edges, N)
        out = torch.empty_like(v)
        lse = torch.empty((N, H), device=dev, dtype=torch.float32)
        p, ip = _lib.ptr, _lib.iptr
        _lib.invoke("cfb200_dpa_fwd", 1, dev, p(q), p(k), p(v), p(a), p(b), ip(edges), ip(e_start), N, E, p(out), p(lse), None)
        res = out[..., :C].contiguous()
        ctx.mark_non_differentiable(res)
        return res

    @staticmethod
    def backward(ctx, go_ihk):
        return None, None, None, None, None, None, None
