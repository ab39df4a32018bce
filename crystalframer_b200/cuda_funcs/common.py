"""Helpers shared by the autograd Functions."""
import weakref

import torch

from .. import _lib

_csr_cache = {}


def csr_offsets(edge_ij_e, N):
    """e_start (N+1): first pair of every query atom.  The reference rebuilds it with
    scatter_add + cumsum in each Function (models/cuda_funcs/fused_dpa.py:24-26); here it is
    computed once per pair list and cached while that tensor is alive and unmodified."""
    key = id(edge_ij_e)
    hit = _csr_cache.get(key)
    if hit is not None:
        ref, version, n, out = hit
        if ref() is edge_ij_e and version == edge_ij_e._version and n == N:
            return out
    E = edge_ij_e.shape[1]
    out = torch.empty(N + 1, dtype=torch.int64, device=edge_ij_e.device)
    _lib.invoke("cfb200_csr_offsets", 1, edge_ij_e.device, _lib.iptr(edge_ij_e), E, N, _lib.iptr(out))
    if len(_csr_cache) > 64:
        for k in [k for k, v in _csr_cache.items() if v[0]() is None]:
            del _csr_cache[k]
    _csr_cache[key] = (weakref.ref(edge_ij_e), edge_ij_e._version, N, out)
    return out


def register_csr(edge_ij_e, N, e_start):
    """Lets a caller that already holds the offsets (cfb200_edge_index) seed the cache."""
    _csr_cache[id(edge_ij_e)] = (weakref.ref(edge_ij_e), edge_ij_e._version, N, e_start)


def f32c(t):
    return None if t is None else t.detach().contiguous().float()
