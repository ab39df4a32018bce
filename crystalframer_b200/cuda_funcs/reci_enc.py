"""autograd Function for the reciprocal-space lattice sum of the plain Crystalformer ("reci", "RECI" and
"multihead" domains)."""
import torch

from .. import _lib
from .common import csr_offsets, f32c


class ReciPeriodicEncodingFuncCUDA(torch.autograd.Function):
    """Drop-in for models/cuda_funcs/reci_space_enc.py:17-97.

    ``forward(a_ik (N,H), kr_base_e (E,3), rvecs_n (B,3,3), vcell_n (B), batch_i (N), edge_ij_e (2,E))`` returns
    ``z_ek (E,H) = log(max(sum_n w exp(a |nG|^2) cos(n . kr), 1e-6)) + 1.5 log(-4 pi a) - log(vcell)``;
    the only gradient is that of ``a_ik`` and, like the reference's, it leaves out the normaliser's
    term (constant over an atom's pairs, so it cancels in the softmax).  ``H`` may differ from the
    configured head count: the "multihead" domain hands over half of the heads
    (models/indexed_lattice_multi_head_attention_cuda.py:953-963)."""

    @staticmethod
    def forward(ctx, a_ik, kr_base_e, rvecs_n, vcell_n, batch_i, edge_ij_e):
        N, H = a_ik.shape
        E = edge_ij_e.shape[1]
        dev = a_ik.device
        a, kr, rv, vc = f32c(a_ik), f32c(kr_base_e), f32c(rvecs_n), f32c(vcell_n)
        batch, edges = batch_i.contiguous(), edge_ij_e.contiguous()
        e_start = csr_offsets(edges, N)
        z = torch.empty((E, H), device=dev, dtype=torch.float32)
        sumexp = torch.empty((E, H), device=dev, dtype=torch.float32)
        p, ip = _lib.ptr, _lib.iptr
        _lib.invoke("cfb200_reci_enc_fwd", 1, dev, p(a), p(kr), p(rv), p(vc), ip(batch), ip(e_start), N, H, E, p(z),
                    p(sumexp))
        ctx.save_for_backward(a, kr, rv, batch, e_start, sumexp)
        return z

    @staticmethod
    def backward(ctx, gz_ek):
        a, kr, rv, batch, e_start, sumexp = ctx.saved_tensors
        N, H = a.shape
        E = kr.shape[0]
        ga = torch.empty_like(a)
        p, ip = _lib.ptr, _lib.iptr
        _lib.invoke("cfb200_reci_enc_bwd", 1, a.device, p(a), p(kr), p(rv), ip(batch), ip(e_start), p(f32c(gz_ek)),
                    p(sumexp), N, H, E, p(ga))
        return ga, None, None, None, None, None
