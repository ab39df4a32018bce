"""The drop-in contract, checked against the reference's own source where its tree is present.

The reference's attention module does ``from .cuda_funcs import *`` and calls the autograd Functions positionally.
Swapping this package's ``cuda_funcs`` in for ``models.cuda_funcs`` therefore needs (i) the reference module to
import with the swapped package, (ii) every Function name it uses on the supported branches to resolve to this
package's class, and (iii) each ``forward`` to take the reference's parameters (same names, same order, same
defaults) and each ``backward`` to return one slot per forward input.  Running the reference module end to end needs
a GPU *and* the reference tree, which do not meet on one machine here; numerical equivalence of the callers is
covered by this package's own mirror of that module (tests/test_gpu_parity.py).  Skipped where the reference tree
is absent.
"""
import ast
import inspect
import os
import sys
import types

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle import build_oracle  # noqa: E402

REF = build_oracle.reference_root()
pytestmark = pytest.mark.skipif(REF is None, reason="reference tree not present (CF_REFERENCE_ROOT)")

# reference file -> Function classes it defines that this package offers as drop-ins
FUNCTIONS = {
    "real_space_framed_proj.py": ["RealEncodingWithFramedProjFuncCUDA"],
    "real_space_enc_proj.py": ["RealPeriodicEncodingWithProjFuncCUDA"],
    "calc_maximum_frame.py": ["ComputeFrame1MaximumMethodCUDA", "ComputeFrame2MaximumMethodCUDA", "ComputeFrame3MaximumMethodCUDA"],
    "calc_maximum_static_frame.py": ["ComputeFrame1MaximumStaticMethodCUDA", "ComputeFrame2MaximumStaticMethodCUDA"],
    "calc_lattice_frame.py": ["ComputeLatticeFrameCUDA"],
    "calc_pca_frame.py": ["ComputePCAFrame"],
    "fused_dpa.py": ["FusedDotProductAttentionCUDA"],
    "fused_dpa_sigmamat.py": ["FusedDotProductAttentionSigmaMatCUDA"],
    "irregular_mean.py": ["IrregularMeanCUDA"],
    "reci_space_enc.py": ["ReciPeriodicEncodingFuncCUDA"],
    "real_space_enc.py": ["RealPeriodicEncodingFuncCUDA"],
}


def _reference_forward_params(path, cls_name):
    """(parameter names without ctx, number of defaults, slots returned by backward) of a reference Function."""
    tree = ast.parse(open(path).read())
    for node in tree.body:
        if isinstance(node, ast.ClassDef) and node.name == cls_name:
            out = {}
            for fn in node.body:
                if isinstance(fn, ast.FunctionDef) and fn.name in ("forward", "backward"):
                    out[fn.name] = fn
            fwd = out["forward"]
            names = [a.arg for a in fwd.args.args][1:]
            n_def = len(fwd.args.defaults)
            slots = None
            for stmt in ast.walk(out["backward"]):
                if isinstance(stmt, ast.Return) and isinstance(stmt.value, ast.Tuple):
                    slots = max(slots or 0, len(stmt.value.elts))
            return names, n_def, slots
    raise AssertionError(f"{cls_name} not found in {path}")


def test_function_signatures_match_the_reference():
    from crystalframer_b200 import cuda_funcs as ours
    for fname, classes in FUNCTIONS.items():
        path = os.path.join(REF, "models", "cuda_funcs", fname)
        for cls_name in classes:
            names, n_def, slots = _reference_forward_params(path, cls_name)
            cls = getattr(ours, cls_name)
            sig = inspect.signature(cls.forward)
            mine = list(sig.parameters)[1:]
            assert mine == names, (cls_name, mine, names)
            my_defaults = [p for p in list(sig.parameters.values())[1:] if p.default is not inspect.Parameter.empty]
            assert len(my_defaults) == n_def, (cls_name, len(my_defaults), n_def)
            assert all(p.default is None for p in my_defaults), cls_name        # the reference's defaults are all None


def test_compile_kernels_signature_matches_the_reference():
    from crystalframer_b200.cuda_funcs import compile_kernels
    tree = ast.parse(open(os.path.join(REF, "models", "cuda_funcs", "kernel_manager.py")).read())
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "compile_kernels")
    assert [a.arg for a in fn.args.args] == list(inspect.signature(compile_kernels).parameters)


def test_reference_attention_module_imports_with_this_package_swapped_in():
    """``models.cuda_funcs`` replaced by this package's ``cuda_funcs``: the reference's attention module must import
    and every Function it names on the supported branches must be this package's class."""
    import crystalframer_b200.cuda_funcs as ours
    saved = {k: sys.modules.get(k) for k in list(sys.modules) if k == "models" or k.startswith("models.")}
    for k in saved:
        del sys.modules[k]
    pkg = types.ModuleType("models")
    pkg.__path__ = [os.path.join(REF, "models")]
    sys.modules["models"] = pkg
    sys.modules["models.cuda_funcs"] = ours
    try:
        import importlib
        mod = importlib.import_module("models.indexed_lattice_multi_head_attention_cuda")
        for classes in FUNCTIONS.values():
            for cls_name in classes:
                if cls_name == "IrregularMeanCUDA":
                    continue                          # used by models/pooling.py, not by the attention module
                assert getattr(mod, cls_name) is getattr(ours, cls_name), cls_name
        assert mod.CUPY_AVAILABLE is True
        # the module class the encoder instantiates, with the constructor this package mirrors
        ref_init = list(inspect.signature(mod.CrystalformerMultiheadAttentionCUDA.__init__).parameters)
        from crystalframer_b200.attention import CrystalformerMultiheadAttentionCUDA
        assert list(inspect.signature(CrystalformerMultiheadAttentionCUDA.__init__).parameters) == ref_init
        ref_fwd = list(inspect.signature(mod.CrystalformerMultiheadAttentionCUDA.forward).parameters)
        assert list(inspect.signature(CrystalformerMultiheadAttentionCUDA.forward).parameters) == ref_fwd
    finally:
        for k in [k for k in sys.modules if k == "models" or k.startswith("models.")]:
            del sys.modules[k]
        sys.modules.update({k: v for k, v in saved.items() if v is not None})


def test_parameter_names_and_shapes_match_the_reference_module():
    """state_dict keys and shapes of the attention module: reference checkpoints must load."""
    import torch
    import crystalframer_b200.cuda_funcs as ours
    from crystalframer_b200.attention import CrystalformerMultiheadAttentionCUDA
    from crystalframer_b200.latticeformer_params import LatticeformerParams
    saved = {k: sys.modules.get(k) for k in list(sys.modules) if k == "models" or k.startswith("models.")}
    for k in saved:
        del sys.modules[k]
    pkg = types.ModuleType("models")
    pkg.__path__ = [os.path.join(REF, "models")]
    sys.modules["models"] = pkg
    sys.modules["models.cuda_funcs"] = ours
    try:
        import importlib
        mod = importlib.import_module("models.indexed_lattice_multi_head_attention_cuda")
        ref_params = importlib.import_module("models.latticeformer_params").LatticeformerParams()
        mine_params = LatticeformerParams()
        for P in (ref_params, mine_params):
            P.domain, P.frame_method = "real", "max"
            P.value_pe_dist_real, P.value_pe_angle_real = 64, 64
        torch.manual_seed(0)
        ref = mod.CrystalformerMultiheadAttentionCUDA(128, 8, params=ref_params)
        mine = CrystalformerMultiheadAttentionCUDA(128, 8, params=mine_params)
        a, b = ref.state_dict(), mine.state_dict()
        assert list(a) == list(b)
        assert all(a[k].shape == b[k].shape for k in a)
        mine.load_state_dict(a)
    finally:
        for k in [k for k in sys.modules if k == "models" or k.startswith("models.")]:
            del sys.modules[k]
        sys.modules.update({k: v for k, v in saved.items() if v is not None})


@pytest.mark.gpu
def test_reference_module_runs_on_this_package():
    """The reference's own attention module, unmodified, with ``models.cuda_funcs`` replaced by this package's
    ``cuda_funcs``, against this package's mirror of it: same state_dict, same inputs, outputs and gradients
    compared.  Needs a GPU and the reference tree on one machine (skipped where either is missing)."""
    import importlib
    import numpy as np
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import crystalframer_b200.cuda_funcs as ours
    from crystalframer_b200 import synth
    from crystalframer_b200.attention import CrystalformerMultiheadAttentionCUDA
    from crystalframer_b200.encoder import build_pair_list, compute_lattice_distances_for_cuda
    from crystalframer_b200.latticeformer_params import LatticeformerParams
    dev = torch.device("cuda:0")
    saved = {k: sys.modules.get(k) for k in list(sys.modules) if k == "models" or k.startswith("models.")}
    for k in saved:
        del sys.modules[k]
    pkg = types.ModuleType("models")
    pkg.__path__ = [os.path.join(REF, "models")]
    sys.modules["models"] = pkg
    sys.modules["models.cuda_funcs"] = ours
    try:
        mod = importlib.import_module("models.indexed_lattice_multi_head_attention_cuda")
        ref_params = importlib.import_module("models.latticeformer_params").LatticeformerParams()
        mine_params = LatticeformerParams()
        for P in (ref_params, mine_params):
            P.domain, P.frame_method = "real", "max"
            P.value_pe_dist_real, P.value_pe_angle_real = 64, 64
            P.symm_break_noise = 0.0
        ours.compile_kernels(2, 8, 16, 64, 64, 16, True, 0, 1.0, 4.0, 1.0, 1.0, 0.0)
        torch.manual_seed(0)
        ref = mod.CrystalformerMultiheadAttentionCUDA(128, 8, params=ref_params).to(dev).train()
        mine = CrystalformerMultiheadAttentionCUDA(128, 8, params=mine_params).to(dev).train()
        mine.load_state_dict(ref.state_dict())
        b = synth.make_workload("cfg1")
        sizes = torch.from_numpy(b.sizes).to(dev)
        pos, tv = torch.from_numpy(b.pos).to(dev), torch.from_numpy(b.trans_vec).to(dev)
        edges, _, batch, _ = build_pair_list(sizes, (b.num_atoms, b.num_pairs))
        pos_ij, dist2_min, tvecs, rvecs, vcell, edges = compute_lattice_distances_for_cuda(pos, batch, tv, sizes, 2)
        x = torch.randn(b.num_atoms, 128, device=dev)
        outs = []
        for m in (ref, mine):
            np.random.seed(3)
            xin = x.clone().requires_grad_(True)
            y, _ = m(xin, xin, xin, batch, batch, edges, pos_ij, dist2_min, tvecs, None, rvecs, vcell, None, False)
            y.square().sum().backward()
            outs.append((y.detach(), xin.grad, {n: p.grad for n, p in m.named_parameters() if p.grad is not None}))
        (y0, gx0, g0), (y1, gx1, g1) = outs
        assert torch.allclose(y0, y1, rtol=1e-5, atol=1e-6) and torch.allclose(gx0, gx1, rtol=1e-4, atol=1e-6)
        assert set(g0) == set(g1)
        for n in g0:
            assert torch.allclose(g0[n], g1[n], rtol=1e-4, atol=1e-6 * float(g0[n].abs().max()) + 1e-9), n
    finally:
        for k in [k for k in sys.modules if k == "models" or k.startswith("models.")]:
            del sys.modules[k]
        sys.modules.update({k: v for k, v in saved.items() if v is not None})


def test_whole_model_state_dict_matches_the_reference():
    """The reference's own ``models.latticeformer.Latticeformer`` (default_jarvis.json), instantiated with this
    package's ``cuda_funcs`` swapped in, against this package's model: same state_dict keys in the same order and the
    same shapes, so the reference's checkpoints load here and vice versa."""
    import importlib
    import json
    import crystalframer_b200.cuda_funcs as ours
    from crystalframer_b200.cuda_funcs import kernel_manager
    from crystalframer_b200.latticeformer import Latticeformer, ModelParams
    saved = {k: sys.modules.get(k) for k in list(sys.modules) if k == "models" or k.startswith("models.")}
    for k in saved:
        del sys.modules[k]
    stubbed = []
    for name in ("torch_scatter", "cupy", "pytorch_pfn_extras", "torch_geometric", "torch_geometric.data", "torch_geometric.nn"):
        if name not in sys.modules:              # imported at module level by the reference, not used on this path
            try:
                importlib.import_module(name)
            except Exception:
                sys.modules[name] = types.ModuleType(name)
                stubbed.append(name)
    pkg = types.ModuleType("models")
    pkg.__path__ = [os.path.join(REF, "models")]
    sys.modules["models"] = pkg
    sys.modules["models.cuda_funcs"] = ours
    kernel_manager.DEFER_BINDING = True          # a parameter container: do not bind constants in the CUDA library
    try:
        lf = importlib.import_module("models.latticeformer")
        with open(os.path.join(REF, "params", "crystalframer", "default_jarvis.json")) as f:
            cfg = json.load(f)
        params = types.SimpleNamespace(**cfg)
        if not hasattr(params, "targets"):
            params.targets = ["e_form"]
        ref = lf.Latticeformer(params)
        mine = Latticeformer(ModelParams())
        a, b = ref.state_dict(), mine.state_dict()
        assert list(a) == list(b)
        assert all(a[k].shape == b[k].shape for k in a)
        mine.load_state_dict(a)
        ref.load_state_dict(b)
        # the head's options (per-atom projection before pooling, normalisation), which no parameter file of the
        # reference switches on, and the reciprocal-space domains
        for over in (dict(pre_pooling_op="w+bn+relu", norm_type="bn", embedding_dim=[96, 64]),
                     dict(pre_pooling_op="w+relu", norm_type="ln", embedding_dim=[128, 32]),
                     dict(pre_pooling_op="relu", norm_type="no"), dict(pooling="max"),
                     dict(domain="real-reci"), dict(domain="multihead", frame_method="no", value_pe_angle_real=0),
                     dict(gauss_state="x"), dict(gauss_state="1"), dict(gauss_state="x-xavier"), dict(gauss_state="q-kdim")):
            cfg2 = dict(cfg, **{k: (list(v) if isinstance(v, list) else v) for k, v in over.items()})
            p2 = types.SimpleNamespace(**cfg2)
            if not hasattr(p2, "targets"):
                p2.targets = ["e_form"]
            ref2 = lf.Latticeformer(p2)
            mine2 = Latticeformer(ModelParams(**{k: (list(v) if isinstance(v, list) else v) for k, v in over.items()}))
            a2, b2 = ref2.state_dict(), mine2.state_dict()
            assert list(a2) == list(b2), (over, [k for k in a2 if k not in b2], [k for k in b2 if k not in a2])
            assert all(a2[k].shape == b2[k].shape for k in a2), over
    finally:
        kernel_manager.DEFER_BINDING = False
        for name in stubbed:
            sys.modules.pop(name, None)
        for k in [k for k in sys.modules if k == "models" or k.startswith("models.")]:
            del sys.modules[k]
        sys.modules.update({k: v for k, v in saved.items() if v is not None})


def test_every_exported_function_of_the_reference_package_is_offered():
    """The names the reference's ``models/cuda_funcs/__init__.py`` exports, read from its source: all but ``Kernel``
    (its holder of a CuPy RawKernel; kernels are prebuilt here) exist in this package."""
    import crystalframer_b200.cuda_funcs as ours
    tree = ast.parse(open(os.path.join(REF, "models", "cuda_funcs", "__init__.py")).read())
    names = None
    for node in tree.body:
        if isinstance(node, ast.Assign) and any(getattr(t, "id", None) == "__all__" for t in node.targets):
            names = [elt.value for elt in node.value.elts]
    assert names, "no __all__ in the reference package"
    missing = [n for n in names if n != "Kernel" and not hasattr(ours, n)]
    assert not missing, missing
    classes = [n for n in names if n.endswith("CUDA") or n == "ComputePCAFrame"]
    assert len(classes) >= 14 and all(hasattr(getattr(ours, n), "apply") for n in classes)
