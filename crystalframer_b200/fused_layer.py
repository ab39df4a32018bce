"""One autograd node and ONE library call per encoder layer and direction.

The reference runs an encoder layer as ~35 separately tracked torch operations plus its CuPy
Functions (models/indexed_latticeformer_encoder.py:848-890 and
models/indexed_lattice_multi_head_attention_cuda.py:737-996) and prepares a batch with ~60 more
(models/indexed_latticeformer_encoder.py:15-32, :175-245).  At 2-3 k atoms per batch the GPU work of
most of those operations is a few microseconds, so the step time is set by host-side dispatch and
autograd bookkeeping.  Here ``cfb200_batch_geometry`` prepares a batch and
``cfb200_encoder_layer_fwd`` / ``_bwd`` run a whole layer -- input projections, Gaussian
coefficients, frames, lattice-sum attention, output projection, residuals, feed-forward block, and in
the backward all data, weight and bias gradients -- with every kernel enqueued from C.

Used by ``CrystalformerEncoderCUDA.forward`` when the layers have the default structure (real-space
domain, "max" or weighted-PCA frames or none, coefficients from q, no dropout, no layer norm, ReLU);
any other configuration takes the operator-by-operator path.

Gradient sink: when a parameter carries ``_cf_grad_sink`` (a tensor of its shape, set by
``optim.FlatAdamW``) the backward ADDS the parameter's gradient into that tensor and reports no
gradient to autograd, so a training step neither allocates per-parameter gradients nor gathers them.
"""
import ctypes
import math

import torch

from . import _lib
from .cuda_funcs.max_frame import _draw_seed

# entry points whose presence in a trace shows that a layer ran through this module
FUSED_FORWARD_CALLS = ("cfb200_encoder_layer_fwd",)
# cut the longest (atom, head) tasks of the attention kernels into chunks (see cfb200_batch_geometry); a switch for
# tests and measurements
SPLIT_TASKS = True
# give every layer a task table when the geometry carries a chunked queue (False: the layers walk the plain queue of
# atoms; a switch for tests)
TASK_TABLE = True
# training forward leaves per-pair value encodings for the backward pass (no second lattice sum); a switch for tests
# and measurements, and for batches whose (E,H,17) floats per layer do not fit
SAVE_PAIR_RESULTS = True
# test hook: a list here receives a copy of every layer's frames (3,N,H,3) as the forward computes them
FRAME_TAP = None
# callable(tensors) invoked by the layer backward right after it has enqueued the kernels that add the layer's
# weight gradients into their sinks (optim.FlatAdamW.overlap_exchange sets it to start the ranks' exchange of
# those slices while the backward pass of the earlier layers runs)
SINKS_FILLED = None

FRAME_METHODS = {"no": 0, "max": 1, "weighted_pca": 2, "max_static": 3, "lattice": 4, "pca": 5}
WEIGHT_FIELDS = ("q_proj", "k_proj", "v_proj", "in_bias", "lattice_pos", "gauss_scale", "out_proj", "out_bias",
                 "pe_dist", "pe_ang1", "pe_ang2", "pe_ang3", "ff1", "ff1_bias", "ff2", "ff2_bias")
GRAD_FIELDS = tuple(f for f in WEIGHT_FIELDS if f != "gauss_scale")


def _align(n, a=64):
    return (n + a - 1) // a * a


class LayerGeometry:
    """Per-batch tensors shared by all layers: pair list, relative positions, reciprocal-vector lengths, the
    per-pair geometry cache (nearest image, smallest squared distance, translations sorted by distance:
    pure geometry, identical for every head and layer), the work-queue order of the attention kernels and
    a scratch buffer that all layers of the batch reuse (their kernels run on one stream, in order)."""

    def __init__(self):
        self.c = _lib.Geometry()
        self.N = self.E = self.B = 0
        self.cache_range = 0
        self._keep = []
        self._ws = None

    @classmethod
    def from_raw(cls, pos, trans, sizes, N, E, cutoff):
        """One call of cfb200_batch_geometry on raw positions (N,3), lattice vectors (B,3,3), sizes (B)."""
        from .cuda_funcs.common import pair_list_fits
        from .cuda_funcs.kernel_manager import KernelManager
        g = cls()
        dev = pos.device
        B = trans.shape[0]
        cfg = KernelManager.config
        rng = int(cfg.lattice_range if cutoff == 0.0 else cfg.minimum_range)
        want_list = rng > 0 and (2 * rng + 1) ** 3 <= 128 and pair_list_fits(E, dev)
        # int64 block: edges (2E) | e_start (N+1) | batch (N) | crystal_start (B+1)
        o_es = 2 * E
        o_b = o_es + N + 1
        o_cs = o_b + N
        ibuf = torch.empty(o_cs + B + 1, dtype=torch.int64, device=dev)
        # float32 block: pos_ij (3E) | rvlen (3B) | pair_cache (4E) | order (queue entries, int32) | counters (64, int32)
        # | chunk records and arrival counters of the queue (int32) | call scratch
        ws_bytes = int(_lib.lib().cfb200_batch_geometry_workspace_bytes(B))
        n_queue, n_split = int(_lib.lib().cfb200_queue_entries(N)), int(_lib.lib().cfb200_split_ints(N))
        o_rv = _align(3 * E)
        o_pc = _align(o_rv + 3 * B)
        o_or = _align(o_pc + 4 * E)
        o_ct = _align(o_or + n_queue)
        o_sp = _align(o_ct + 64)
        o_ws = _align(o_sp + n_split)
        fbuf = torch.empty(o_ws + ws_bytes // 4, dtype=torch.float32, device=dev)
        plist = torch.empty((E, 5, 128), dtype=torch.float32, device=dev) if want_list else None
        ip, fp = ibuf.data_ptr(), fbuf.data_ptr()
        _lib.invoke("cfb200_batch_geometry", 7, dev, _lib.ptr(pos), _lib.ptr(trans), _lib.iptr(sizes), B, N, E, rng,
                    ip, ip + 8 * o_es, ip + 8 * o_b, ip + 8 * o_cs, fp, None, fp + 4 * o_rv, None,
                    fp + 4 * o_pc if rng > 0 else None, _lib.ptr(plist), fp + 4 * o_or, fp + 4 * o_sp if SPLIT_TASKS else None,
                    fp + 4 * o_ws, ws_bytes)
        g.N, g.E, g.B, g.cache_range = N, E, B, rng
        g._keep = [ibuf, fbuf, plist, pos, trans, sizes]
        g.edges = ibuf[:2 * E].view(2, E)
        g.e_start = ibuf[o_es:o_es + N + 1]
        g.batch = ibuf[o_b:o_b + N]
        g.pos_ij = fbuf[:3 * E].view(E, 3)
        g.rvlen = fbuf[o_rv:o_rv + 3 * B].view(B, 3)
        g.tvecs = trans
        c = g.c
        c.pos_ij, c.tvecs, c.rvlen = fp, trans.data_ptr(), fp + 4 * o_rv
        c.batch, c.edges, c.e_start = ip + 8 * o_b, ip, ip + 8 * o_es
        c.order, c.counters = fp + 4 * o_or, fp + 4 * o_ct
        c.split = fp + 4 * o_sp if SPLIT_TASKS else None
        g.split = fbuf[o_sp:o_sp + n_split].view(torch.int32) if SPLIT_TASKS else None
        c.pair_cache = fp + 4 * o_pc if rng > 0 else None
        c.pair_list = plist.data_ptr() if plist is not None else None
        c.N, c.E, c.cache_range = N, E, g.cache_range
        return g

    @classmethod
    def from_tensors(cls, pos_ij, tvecs, batch, edges, rvlen, cutoff=0.0):
        """From the tensors the reference's callers hand to a layer (pair list and relative positions already
        built): adds CSR offsets, the per-pair geometry cache and the work-queue order."""
        from .cuda_funcs.common import csr_offsets, pair_geometry
        g = cls()
        g.N, g.E, g.B = batch.shape[0], edges.shape[1], tvecs.shape[0]
        g.pos_ij, g.tvecs, g.batch, g.edges, g.rvlen = pos_ij, tvecs, batch, edges, rvlen
        g.e_start = csr_offsets(edges, g.N)
        pair_cache, pair_list, g.cache_range = pair_geometry(pos_ij, tvecs, batch, edges, cutoff)
        pairs_per_atom = (g.e_start[1:] - g.e_start[:-1]).float()
        vcell = (tvecs[:, 0] * torch.linalg.cross(tvecs[:, 1], tvecs[:, 2])).sum(1).abs().clamp_min(1e-6)
        survivors = (2145.0 / vcell).clamp(1.0, 125.0)[batch]
        order = torch.argsort(pairs_per_atom * (7.0 + survivors), descending=True, stable=True).to(torch.int32)
        counters = torch.zeros(64, dtype=torch.int32, device=pos_ij.device)
        g._keep = [pair_cache, pair_list, order, counters]
        c = g.c
        c.pos_ij, c.tvecs, c.rvlen = _lib.ptr(pos_ij), _lib.ptr(tvecs), _lib.ptr(rvlen)
        c.batch, c.edges, c.e_start = _lib.iptr(batch), _lib.iptr(edges), _lib.iptr(g.e_start)
        c.order, c.counters = order.data_ptr(), counters.data_ptr()
        c.pair_cache, c.pair_list = _lib.ptr(pair_cache), _lib.ptr(pair_list)
        c.N, c.E, c.cache_range = g.N, g.E, g.cache_range
        c.split = None
        return g

    def workspace(self, nbytes, device):
        if self._ws is None or self._ws.numel() < nbytes:
            self._ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)
        return self._ws


def _state_layout(N, E, H, D, F, frames, tasks_bytes=0, pair_results=False):
    """Offsets (floats) of the activations a layer's forward leaves for its backward, in one buffer.
    ``pair_results``: room for the per-pair value encodings (val, px, upool) with which the backward pass needs no
    second lattice sum."""
    hd = D // H
    sizes = (("q", N * D), ("q_scaled", N * D), ("k", N * D), ("v", N * D), ("a", N * H),
             ("frames", 9 * N * H if frames else 0), ("z", E * H), ("spool", N * H * 256), ("attn", N * D),
             ("lse", N * H), ("x1", N * D), ("h", N * F), ("tasks", tasks_bytes // 4),
             ("val", E * H * hd if pair_results else 0), ("px", E * H if pair_results else 0),
             ("upool", N * D if pair_results else 0))
    off, total = {}, 0
    for name, n in sizes:
        off[name] = total if n else None
        total += _align(n)
    return off, total


class FusedEncoderLayerFunc(torch.autograd.Function):
    """forward(x, q_proj, k_proj, v_proj, in_bias, lattice_pos, gauss_scale, out_proj, out_bias, pe_dist, pe_ang1,
    pe_ang2, pe_ang3, ff1, ff1_bias, ff2, ff2_bias, geometry, meta) -> x_out"""

    @staticmethod
    def forward(ctx, x, *args):
        params, geo, meta = args[:16], args[16], args[17]
        H, hd, F = meta["H"], meta["hd"], meta["F"]
        N, E, dev = geo.N, geo.E, x.device
        D = H * hd
        x = x.contiguous()
        method = FRAME_METHODS[meta["frame_method"]]
        if method == 2:
            # weighted-PCA frames: the same draws from the generators as cuda_funcs.weighted_pca_frames
            _draw_seed()
            seed1 = _draw_seed()
            seed2 = int(torch.randint(0, 2 ** 62, (1,)).item())
        elif method in (1, 3):
            seed1, seed2 = _draw_seed(), _draw_seed()
        elif method == 4:
            seed1, seed2 = _draw_seed(), _draw_seed()
            _draw_seed()                       # the reference draws three seeds for its three lattice kernels
        elif method == 5:
            seed1, seed2 = int(torch.randint(0, 2 ** 62, (1,)).item()), 0      # as cuda_funcs.ComputePCAFrame
        else:
            seed1 = seed2 = 0
        desc = _lib.LayerDesc(D, F, method, meta["lb"], meta["beta"], meta["scale_real"], meta["dist_max"], meta["cutoff"],
                              seed1, seed2)
        W = _lib.LayerWeights(*[None if p is None else _lib.ptr(p) for p in params])
        tasks_bytes = int(_lib.lib().cfb200_attn_tasks_bytes(N)) if geo.c.split and TASK_TABLE else 0
        # with gradients wanted the forward stores per-pair results (68 bytes per pair and head) and the backward
        # needs no second lattice sum; without, the lighter forward runs
        save_pairs = SAVE_PAIR_RESULTS and any(ctx.needs_input_grad)
        off, total = _state_layout(N, E, H, D, F, method != 0, tasks_bytes, save_pairs)
        state = torch.empty(total, dtype=torch.float32, device=dev)
        base = state.data_ptr()
        St = _lib.LayerState(*[None if off[f] is None else base + 4 * off[f] for f, _ in _lib.LayerState._fields_])
        out = torch.empty_like(x)
        nbytes = int(_lib.lib().cfb200_encoder_layer_workspace_bytes(N, E, D, F, method))
        ws = geo.workspace(nbytes, dev)
        _lib.invoke("cfb200_encoder_layer_fwd", 8 + (method in (1, 3, 4, 5)) + 2 * (method == 2), dev, ctypes.byref(desc),
                    ctypes.byref(W), ctypes.byref(geo.c), x.data_ptr(), ctypes.byref(St), out.data_ptr(), ws.data_ptr(),
                    ws.numel())
        if FRAME_TAP is not None and method != 0:
            FRAME_TAP.append(state[off["frames"]:off["frames"] + 9 * N * H].view(3, N, H, 3).clone())
        ctx.save_for_backward(x, state, *params)
        ctx.geo, ctx.desc, ctx.St, ctx.W = geo, desc, St, W
        ctx.sinks = tuple(getattr(p, "_cf_grad_sink", None) if p is not None else None for p in params)
        return out

    @staticmethod
    def backward(ctx, g):
        x, state = ctx.saved_tensors[:2]
        params = ctx.saved_tensors[2:]
        geo, desc = ctx.geo, ctx.desc
        N, E, dev = geo.N, geo.E, x.device
        g = g.contiguous()
        gx = torch.empty_like(x)
        named = dict(zip(WEIGHT_FIELDS, params))
        sinks = dict(zip(WEIGHT_FIELDS, ctx.sinks))
        trainable = [f for f in GRAD_FIELDS if named[f] is not None]
        use_sink = all(sinks[f] is not None for f in trainable)
        if use_sink:
            dest = {f: sinks[f] for f in trainable}
        else:
            # one buffer for all gradients of the layer, handed to autograd as views
            offs, total = {}, 0
            for f in trainable:
                offs[f] = total
                total += _align(named[f].numel())
            flat = torch.empty(total, dtype=torch.float32, device=dev)
            dest = {f: flat[offs[f]:offs[f] + named[f].numel()].view(named[f].shape) for f in trainable}
        Gr = _lib.LayerGrads(*[dest[f].data_ptr() if f in dest else None for f in GRAD_FIELDS])
        nbytes = int(_lib.lib().cfb200_encoder_layer_workspace_bytes(N, E, desc.d_model, desc.ff_dim, desc.frame_method))
        ws = geo.workspace(nbytes, dev)
        _lib.invoke("cfb200_encoder_layer_bwd", 9 + (1 if use_sink else 0), dev, ctypes.byref(desc), ctypes.byref(ctx.W),
                    ctypes.byref(geo.c), x.data_ptr(), ctypes.byref(ctx.St), g.data_ptr(), gx.data_ptr(),
                    ctypes.byref(Gr), 1 if use_sink else 0, ws.data_ptr(), ws.numel())
        if use_sink:
            grads = [None] * 16
            if SINKS_FILLED is not None:
                SINKS_FILLED(tuple(dest.values()))       # this layer's gradients are final (enqueued): they may be exchanged
        else:
            grads = [dest.get(f) for f in WEIGHT_FIELDS]
        return (gx, *grads, None, None)


def layer_meta(layer):
    """Scalars of an encoder layer in the form the Function takes; None if the layer's configuration is
    outside what the fused path covers."""
    attn = layer.self_attn
    P = attn.params
    if P.domain != "real" or P.frame_method not in FRAME_METHODS or P.gauss_state != "q" or not P.normalize_gauss:
        return None
    if attn.in_proj_bias is None or attn.pe_dist_proj is None or attn.dropout != 0.0:
        return None
    if (attn.proj_angle1 is None) != (P.frame_method == "no"):
        return None                      # angle weights exactly when there are frames
    if attn.kdim != attn.embed_dim or attn.vdim != attn.embed_dim:
        return None
    if layer.linear1.bias is None or layer.linear2.bias is None or layer.linear1.out_features % 4:
        return None
    dist_max = P.value_pe_dist_max
    if dist_max < 0:
        dist_max = (-dist_max) * P.scale_real
    if P.adaptive_cutoff_sigma < 0:
        cutoff = float(P.adaptive_cutoff_sigma)
    elif P.adaptive_cutoff_sigma > 0:
        cutoff = float(P.scale_real * P.gauss_lb_real ** (-0.5) * P.adaptive_cutoff_sigma)
    else:
        cutoff = 0.0
    return dict(frame_method=P.frame_method, H=attn.num_heads, hd=attn.head_dim, F=layer.linear1.out_features,
                lb=float(P.gauss_lb_real), beta=float(P.positive_func_beta), scale_real=float(P.scale_real),
                dist_max=float(dist_max), cutoff=cutoff)


def layer_parameters(layer):
    """The layer's parameters in the Function's order (WEIGHT_FIELDS)."""
    attn = layer.self_attn
    pe = lambda p: None if p is None else p
    return (attn.q_proj_weight, attn.k_proj_weight, attn.v_proj_weight, attn.in_proj_bias, attn.lattice_pos_weights,
            attn.gauss_scale, attn.out_proj.weight, attn.out_proj.bias, pe(attn.pe_dist_proj), pe(attn.proj_angle1),
            pe(attn.proj_angle2), pe(attn.proj_angle3), layer.linear1.weight, layer.linear1.bias, layer.linear2.weight,
            layer.linear2.bias)
