"""Inference with checkpoints written by the reference's training module.

The reference's Lightning module (models/regression.py:30-59) saves the live model under ``model.*``, the running
weight average under ``swa_model.module.*`` (plus ``swa_model.n_averaged``) and the target statistics in the
buffers ``target_std`` / ``target_mean``; its demo (demo.py:67-88) loads the averaged weights and folds the
statistics into the last linear layer, so that the network predicts in the targets' own units.  The model of this
package has the reference's state_dict (tests/test_dropin_contract.py), so those checkpoints load unchanged."""
import torch

from .latticeformer import Latticeformer, ModelParams


def load_reference_checkpoint(model: Latticeformer, checkpoint, prefix="swa_model.module.", denormalize=True):
    """Loads a reference checkpoint (the dict ``torch.load`` returns, or its ``state_dict``) into ``model``.

    ``prefix``: ``"swa_model.module."`` for the averaged weights (what demo.py evaluates), ``"model."`` for the live
    ones.  ``denormalize``: scale the last linear layer by ``target_std`` and shift it by ``target_mean`` as
    demo.py:84-88 does.  Returns ``(target_std, target_mean)``."""
    state = checkpoint.get("state_dict", checkpoint)
    picked = {k[len(prefix):]: v for k, v in state.items() if k.startswith(prefix)}
    if not picked:
        raise KeyError(f"no entry of the checkpoint starts with {prefix!r}")
    model.load_state_dict(picked)
    std, mean = state["target_std"], state["target_mean"]
    if denormalize:
        last = model.mlp[-1]
        with torch.no_grad():
            std_d, mean_d = std.to(last.weight), mean.to(last.weight)
            last.bias.copy_(last.bias * std_d + mean_d)
            last.weight.copy_(last.weight * std_d[:, None])
    # the loaded gauss_scale is picked up by attention.gauss_scale_ready (an in-place load moves the tensor's version)
    return std, mean


def reference_checkpoint_of(model: Latticeformer, averaged_state=None, target_std=None, target_mean=None, n_averaged=1):
    """The reference's checkpoint layout for ``model`` (for tests and for handing weights trained here to the
    reference's demo): ``{"state_dict": {"model.*", "swa_model.module.*", "swa_model.n_averaged", "target_std",
    "target_mean"}}``.  ``averaged_state``: state_dict of the averaged weights (default: the live ones)."""
    live = {k: v.detach().cpu().clone() for k, v in model.state_dict().items()}
    avg = live if averaged_state is None else {k: v.detach().cpu().clone() for k, v in averaged_state.items()}
    n_out = model.mlp[-1].out_features
    state = {f"model.{k}": v for k, v in live.items()}
    state.update({f"swa_model.module.{k}": v for k, v in avg.items()})
    state["swa_model.n_averaged"] = torch.tensor(n_averaged)
    state["target_std"] = torch.ones(n_out) if target_std is None else torch.as_tensor(target_std, dtype=torch.float32)
    state["target_mean"] = torch.zeros(n_out) if target_mean is None else torch.as_tensor(target_mean, dtype=torch.float32)
    return {"state_dict": state}


@torch.no_grad()
def evaluate(model: Latticeformer, batches):
    """Mean absolute error per target over device-resident batches (demo.py:104-121): the model in eval mode, no
    gradients (the lighter forward kernels), predictions compared with ``batch.y``.  Returns ``(mae (T,),
    predictions (sum B, T))``."""
    was_training = model.training
    model.eval()
    outs, errs = [], []
    for tb in batches:
        out = model(tb)
        outs.append(out)
        errs.append((out - tb.y).abs())
    if was_training:
        model.train()
    return torch.cat(errs).mean(0), torch.cat(outs)


def build_model(**overrides):
    """Model with the reference's default_jarvis.json hyper-parameters, overridden by keyword."""
    return Latticeformer(ModelParams(**overrides))
