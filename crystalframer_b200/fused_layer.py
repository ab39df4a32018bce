"""One autograd Function for a whole encoder layer.

The reference runs an encoder layer as ~35 separately tracked torch operations plus its CuPy
Functions (models/indexed_latticeformer_encoder.py:848-890 and
models/indexed_lattice_multi_head_attention_cuda.py:737-996).  At 2-3 k atoms per batch the
GPU work of most of those operations is a few microseconds, so the step time is set by host-side
dispatch and autograd bookkeeping.  This Function performs the same arithmetic -- input
projections, Gaussian coefficients, max frames, lattice-sum bias and value encoding, ragged
attention, output projection, residuals and the feed-forward block -- with one graph node: the
dense layers stay on cuBLAS through ``torch.addmm`` / ``torch.mm``, everything specific to the
periodic attention runs in libcfb200, and the backward pass is written out by hand.

Used by ``CrystalformerEncoderLayerCUDA.forward`` when the layer has the default structure
(real-space domain, "max" or weighted-PCA frames or none, coefficients from q, no dropout, no layer norm, ReLU); any other
configuration takes the operator-by-operator path.
"""
import math

import torch

from . import _lib
from .cuda_funcs.common import csr_offsets, pair_geometry
from .cuda_funcs.max_frame import _draw_seed


FUSED_ATTENTION = True      # lattice sums + attention as one kernel per direction; False: separate entry points

_side_streams = {}


def _side_stream(dev):
    """Second stream of a device for work that does not sit on the layer's critical path (weight and
    bias gradients): those GEMMs fill half of the SMs, so they run beside the data-gradient chain."""
    s = _side_streams.get(dev)
    if s is None:
        s = _side_streams[dev] = torch.cuda.Stream(device=dev)
    return s


class LayerGeometry:
    """Per-batch tensors shared by all layers, and the per-pair geometry cache (nearest image and
    smallest squared distance of every pair): pure geometry, the same for every head and layer, so it
    is computed once per batch for the lattice range nearly all (atom, head) pairs end up with."""
    __slots__ = ("pos_ij", "tvecs", "batch", "edges", "e_start", "rvlen", "N", "E", "pair_cache", "pair_list",
                 "cache_range", "order", "counters")

    def __init__(self, pos_ij, tvecs, batch, edges, rvlen, cutoff=0.0):
        self.pos_ij, self.tvecs, self.batch, self.edges, self.rvlen = pos_ij, tvecs, batch, edges, rvlen
        self.N, self.E = batch.shape[0], edges.shape[1]
        self.e_start = csr_offsets(edges, self.N)
        self.pair_cache, self.pair_list, self.cache_range = pair_geometry(pos_ij, tvecs, batch, edges, cutoff)
        # The order in which the per-atom attention kernels hand out work: most expensive atoms first.  An
        # atom costs about (a constant + its surviving translations) per pair, and the translations within
        # reach of a Gaussian of typical width number about (a sphere of radius 8 A) / (cell volume).
        pairs_per_atom = (self.e_start[1:] - self.e_start[:-1]).float()
        vcell = (tvecs[:, 0] * torch.linalg.cross(tvecs[:, 1], tvecs[:, 2])).sum(1).abs().clamp_min(1e-6)
        survivors = (2145.0 / vcell).clamp(1.0, 125.0)[batch]
        self.order = torch.argsort(pairs_per_atom * (7.0 + survivors), descending=True, stable=True).to(torch.int32)
        self.counters = torch.zeros(64, dtype=torch.int32, device=pos_ij.device)


class FusedEncoderLayerFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, Wq, Wk, Wv, b_in, w_lat, gauss_scale, Wo, bo, Wd, W1, W2, W3, Wf1, bf1, Wf2, bf2, geo, meta):
        H, hd = meta["H"], meta["hd"]
        N, E, dev = geo.N, geo.E, x.device
        D = H * hd
        p, ip = _lib.ptr, _lib.iptr
        x = x.contiguous()
        bq, bk, bv = b_in[:D], b_in[D:2 * D], b_in[2 * D:]
        q = torch.addmm(bq, x, Wq.t())
        k = torch.addmm(bk, x, Wk.t())
        v = torch.addmm(bv, x, Wv.t())
        new = lambda *shape: torch.empty(shape, device=dev, dtype=torch.float32)
        a, qs = new(N, H), new(N, H, hd)
        _lib.invoke("cfb200_gauss_coef_fwd", 1, dev, p(q), p(w_lat), p(gauss_scale), N, meta["lb"], meta["beta"],
                    meta["scale_real"], p(a), p(qs))
        plain = meta["frame_method"] == "no"           # plain Crystalformer: un-windowed distance encoding, no frames
        f = None if plain else new(3, N, H, 3)
        fr = (None, None, None) if plain else (f[0], f[1], f[2])
        if plain:
            pass
        elif meta["frame_method"] == "max":
            s1, s2 = _draw_seed(), _draw_seed()
            _lib.invoke("cfb200_max_frames_cached", 1, dev, p(qs), p(k), p(a), p(geo.pos_ij), p(geo.tvecs), p(geo.rvlen),
                        ip(geo.batch), ip(geo.edges), ip(geo.e_start), N, E, meta["cutoff"], s1, s2, p(f[0]), p(f[1]),
                        p(f[2]), p(geo.pair_cache), p(geo.pair_list), geo.cache_range)
        else:
            # weighted-PCA frames; the same draws from the generators as cuda_funcs.weighted_pca_frames
            _draw_seed()
            seed_noise = _draw_seed()
            seed_sign = int(torch.randint(0, 2 ** 62, (1,)).item())
            nbytes = int(_lib.lib().cfb200_sigma_frames_workspace_bytes(N, E))
            ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=dev)
            _lib.invoke("cfb200_sigma_frames", 2, dev, p(qs), p(k), p(a), p(geo.pos_ij), p(geo.tvecs), p(geo.rvlen),
                        ip(geo.batch), ip(geo.edges), ip(geo.e_start), N, E, meta["cutoff"], seed_noise, seed_sign,
                        p(f[0]), p(f[1]), p(f[2]), ws.data_ptr(), nbytes)
        Wd3 = Wd[0]
        W13, W23, W33 = (None, None, None) if plain else (W1[0], W2[0], W3[0])
        o, lse = new(N, H, hd), new(N, H)
        if FUSED_ATTENTION or plain:
            # lattice sums, value encoding and attention in one kernel: the basis sums are pooled with the
            # attention weights and projected once per (atom, head)
            z, val, spool = new(E, H), None, new(N, H, 4 * 64)
            _lib.invoke("cfb200_attn_fused_fwd", 1, dev, p(qs), p(k), p(v), p(a), p(geo.pos_ij), p(geo.tvecs),
                        p(geo.rvlen), ip(geo.batch), ip(geo.edges), ip(geo.e_start), p(geo.order, torch.int32),
                        p(geo.counters, torch.int32), N, E,
                        meta["dist_max"], meta["cutoff"], p(Wd3), p(W13), p(W23), p(W33), p(fr[0]), p(fr[1]), p(fr[2]),
                        p(geo.pair_list), geo.cache_range, p(o), p(z), p(lse), p(spool), 1 if plain else 0)
        else:
            z, val, spool = new(E, H), new(E, H, hd), None
            _lib.invoke("cfb200_framed_proj_fwd_cached", 1, dev, p(a), p(geo.pos_ij), p(geo.tvecs), p(geo.rvlen),
                        ip(geo.batch), ip(geo.edges), N, E, meta["dist_max"], meta["cutoff"], p(Wd3), p(W13), p(W23),
                        p(W33), p(f[0]), p(f[1]), p(f[2]), p(z), p(val), p(geo.pair_cache), p(geo.pair_list),
                        geo.cache_range)
            _lib.invoke("cfb200_dpa_fwd", 1, dev, p(qs), p(k), p(v), p(z), p(val), ip(geo.edges), ip(geo.e_start), N, E,
                        p(o), p(lse), None)
        x1 = torch.addmm(bo, o.view(N, D), Wo.t()).add_(x)
        h = torch.addmm(bf1, x1, Wf1.t()).relu_()
        x2 = torch.addmm(bf2, h, Wf2.t()).add_(x1)
        ctx.save_for_backward(x, Wq, Wk, Wv, w_lat, gauss_scale, Wo, Wd, W1, W2, W3, Wf1, Wf2, q, qs, k, v, a, f, z,
                              val if val is not None else spool, o, lse, x1, h)
        ctx.geo, ctx.meta, ctx.fused_attention = geo, meta, val is None
        return x2

    @staticmethod
    def backward(ctx, g):
        (x, Wq, Wk, Wv, w_lat, gauss_scale, Wo, Wd, W1, W2, W3, Wf1, Wf2, q, qs, k, v, a, f, z, val, o, lse, x1,
         h) = ctx.saved_tensors                  # val: the value encoding, or the pooled basis sums (fused attention)
        geo, meta = ctx.geo, ctx.meta
        H, hd = meta["H"], meta["hd"]
        N, E, dev = geo.N, geo.E, x.device
        D = H * hd
        plain = meta["frame_method"] == "no"
        p, ip = _lib.ptr, _lib.iptr
        new = lambda *shape: torch.empty(shape, device=dev, dtype=torch.float32)
        g = g.contiguous()
        main, side = torch.cuda.current_stream(dev), _side_stream(dev)
        # Data gradients run on the current stream; weight and bias gradients, which nothing in this
        # backward pass reads, follow on the side stream as soon as their operands exist.  Every operand
        # stays referenced until the streams are joined at the end, so no block is recycled early.
        ev = torch.cuda.Event()
        ev.record(main)
        gh = torch.ops.aten.threshold_backward(g.mm(Wf2), h, 0)
        gx1 = torch.addmm(g, gh, Wf1)
        ev1 = torch.cuda.Event()
        ev1.record(main)
        go = gx1.mm(Wo)
        with torch.cuda.stream(side):
            side.wait_event(ev)
            gWf2 = g.t().mm(h)
            gbf2 = g.sum(0)
            side.wait_event(ev1)
            gWf1 = gh.t().mm(x1)
            gbf1 = gh.sum(0)
            gWo = gx1.t().mm(o.view(N, D))
            gbo = gx1.sum(0)
        # attention, lattice sums, coefficients
        ga = new(N, H)
        if ctx.fused_attention:
            spool = val
            gqs, gk, gv, gz = new(N, H, hd), new(N, H, hd), new(N, H, hd), new(E, H)
            go = go.view(N, H, hd)
            _lib.invoke("cfb200_attn_fused_bwd", 2, dev, p(qs), p(k), p(v), p(a), p(geo.pos_ij), p(geo.tvecs),
                        p(geo.rvlen), ip(geo.batch), ip(geo.edges), ip(geo.e_start), p(geo.order, torch.int32),
                        p(geo.counters, torch.int32), N, E,
                        meta["dist_max"], meta["cutoff"], p(Wd[0]), *((None,) * 6 if plain else
                                                                      (p(W1[0]), p(W2[0]), p(W3[0]), p(f[0]), p(f[1]), p(f[2]))),
                        p(geo.pair_list), geo.cache_range, p(o), p(z), p(lse), p(go), p(gqs), p(gk), p(gv),
                        p(ga), p(gz), 1 if plain else 0)
            ev3 = torch.cuda.Event()
            ev3.record(main)
            with torch.cuda.stream(side):
                # weight gradients of the value encoding: gW[h] (16 x 256) = sum_i gout[i,h,:]^T spool[i,h,:]
                side.wait_event(ev3)
                gW_all = torch.bmm(go.permute(1, 2, 0), spool.permute(1, 0, 2))
                gW = [gW_all[:, :, 64 * b:64 * (b + 1)].contiguous() for b in range(1 if plain else 4)]
        else:
            gqs, gk, gv, gz, gval = new(N, H, hd), new(N, H, hd), new(N, H, hd), new(E, H), new(E, H, hd)
            _lib.invoke("cfb200_dpa_bwd", 2, dev, p(qs), p(k), p(v), p(z), p(val), ip(geo.edges), ip(geo.e_start), N, E,
                        p(o), p(lse), p(go), p(gqs), p(gk), p(gv), p(gz), p(gval))
            gW = [torch.empty_like(W[0]) for W in (Wd, W1, W2, W3)]
            lib = _lib.lib()
            nbytes = int(lib.cfb200_framed_proj_bwd_workspace_bytes(N, E))
            ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=dev)
            _lib.invoke("cfb200_framed_proj_bwd_cached", 3, dev, p(a), p(geo.pos_ij), p(geo.tvecs), p(geo.rvlen),
                        ip(geo.batch), ip(geo.edges), ip(geo.e_start), N, E, meta["dist_max"], meta["cutoff"], p(Wd[0]),
                        p(W1[0]), p(W2[0]), p(W3[0]), p(f[0]), p(f[1]), p(f[2]), p(z), p(gz), p(gval), p(ga), p(gW[0]),
                        p(gW[1]), p(gW[2]), p(gW[3]), ws.data_ptr(), nbytes, p(geo.pair_list), geo.cache_range)
        gq, gw = new(N, H, hd), torch.empty_like(w_lat)
        _lib.invoke("cfb200_gauss_coef_bwd", 1, dev, p(q), p(w_lat), p(gauss_scale), N, meta["lb"], meta["beta"],
                    meta["scale_real"], p(ga), p(gqs), p(gq), p(gw))
        # input projections
        gq2, gk2, gv2 = gq.view(N, D), gk.view(N, D), gv.view(N, D)
        ev2 = torch.cuda.Event()
        ev2.record(main)
        gx = torch.addmm(gx1, gq2, Wq).addmm_(gk2, Wk).addmm_(gv2, Wv)
        with torch.cuda.stream(side):
            side.wait_event(ev2)
            gWq, gWk, gWv = gq2.t().mm(x), gk2.t().mm(x), gv2.t().mm(x)
            gb_in = torch.cat([gq2.sum(0), gk2.sum(0), gv2.sum(0)])
            done = torch.cuda.Event()
            done.record(side)
        main.wait_event(done)
        for t in (gWf2, gbf2, gWf1, gbf1, gWo, gbo, gWq, gWk, gWv, gb_in) + (tuple(gW) if ctx.fused_attention else ()):
            t.record_stream(main)               # allocated on the side stream, consumed on the current one
        gWa = (None, None, None) if plain else (gW[1].unsqueeze(0), gW[2].unsqueeze(0), gW[3].unsqueeze(0))
        return (gx, gWq, gWk, gWv, gb_in, gw, None, gWo, gbo, gW[0].unsqueeze(0), *gWa, gWf1, gbf1, gWf2, gbf2, None, None)


def layer_meta(attn):
    """Scalars of the attention module in the form the Function takes; None if the layer's
    configuration is outside what the fused path covers."""
    P = attn.params
    if P.domain != "real" or P.frame_method not in ("max", "weighted_pca", "no") or P.gauss_state != "q" or \
            not P.normalize_gauss:
        return None
    if attn.in_proj_bias is None or attn.pe_dist_proj is None or attn.dropout != 0.0:
        return None
    if (attn.proj_angle1 is None) != (P.frame_method == "no"):
        return None                      # angle weights exactly when there are frames
    if attn.kdim != attn.embed_dim or attn.vdim != attn.embed_dim:
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
    return dict(frame_method=P.frame_method, H=attn.num_heads, hd=attn.head_dim, lb=float(P.gauss_lb_real),
                beta=float(P.positive_func_beta), scale_real=float(P.scale_real), dist_max=float(dist_max), cutoff=cutoff)
