"""
Checkpoint interchange with the reference implementation itself. A child process whose import path holds ONLY the
reference install (``baseline/_ref`` plus its three pure-Python stand-in dependencies) writes a checkpoint that this
package loads, and loads a checkpoint that this package wrote. Skipped where the reference is not installed.
"""

import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch

REPO = Path(__file__).resolve().parent.parent
REF = REPO / "baseline" / "_ref"
SHIMS = REPO / "baseline" / "shims"

pytestmark = pytest.mark.skipif(not (REF / "olmo_core").is_dir(), reason="the reference is not installed under baseline/_ref")


def _run_reference(code: str, cwd: Path) -> None:
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([str(SHIMS), str(REF)])
    env.pop("RANK", None)
    env.pop("WORLD_SIZE", None)
    proc = subprocess.run([sys.executable, "-c", textwrap.dedent(code)], cwd=str(cwd), env=env, capture_output=True,
                          text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]


_REF_PRELUDE = """
    import torch, olmo_core
    assert "baseline/_ref" in olmo_core.__file__.replace("\\\\", "/"), olmo_core.__file__
    from olmo_core.nn.transformer import TransformerConfig
    from olmo_core.optim import AdamWConfig
    from olmo_core.distributed.checkpoint import save_model_and_optim_state, load_model_and_optim_state
    torch.manual_seed(0)
    model = TransformerConfig.olmo2_30M(vocab_size=512, n_layers=2).build(init_device="cpu")
    model.init_weights(device=torch.device("cpu"), max_seq_len=64)
    optim = AdamWConfig(lr=2e-3, weight_decay=0.03).build(model)
"""


def _ours(seed):
    from olmo_core_b200.nn.transformer import TransformerConfig
    from olmo_core_b200.optim import AdamWConfig

    torch.manual_seed(seed)
    model = TransformerConfig.olmo2_30M(vocab_size=512, n_layers=2).build(init_device="cpu")
    model.init_weights(max_seq_len=64, device=torch.device("cpu"))
    return model, AdamWConfig(lr=1.0, weight_decay=0.5).build(model)


def test_load_checkpoint_written_by_the_reference(tmp_path):
    from olmo_core_b200.distributed.checkpoint import load_model_and_optim_state

    _run_reference(_REF_PRELUDE + """
    ids = torch.randint(0, 512, (2, 16))
    model(ids, labels=ids).loss.backward()
    optim.step()
    save_model_and_optim_state("ckpt", model, optim, save_overwrite=True)
    torch.save({"params": {n: p.detach().clone() for n, p in model.named_parameters()},
                "exp_avg": {n: optim.state[p]["exp_avg"].clone() for n, p in model.named_parameters()},
                "step": float(next(iter(optim.state.values()))["step"])}, "full.pt")
    """, tmp_path)
    want = torch.load(tmp_path / "full.pt", weights_only=False)
    model, optim = _ours(5)
    load_model_and_optim_state(str(tmp_path / "ckpt"), model, optim)
    assert optim.param_groups[0]["lr"] == pytest.approx(2e-3) and optim.param_groups[0]["weight_decay"] == pytest.approx(0.03)
    for n, p in model.named_parameters():
        assert torch.equal(p.data, want["params"][n]), n
        assert torch.equal(optim.state[p]["exp_avg"], want["exp_avg"][n]), n
        assert float(optim.state[p]["step"]) == want["step"]
    # and the model computes what the reference's computed
    ids = torch.arange(32).view(2, 16) % 512
    torch.save(ids, tmp_path / "ids.pt")
    ours = model(ids).detach() if not hasattr(model(ids), "logits") else model(ids).logits.detach()
    torch.save(ours, tmp_path / "ours_logits.pt")
    _run_reference(_REF_PRELUDE + """
    load_model_and_optim_state("ckpt", model, optim)
    ids = torch.load("ids.pt")
    out = model(ids)
    logits = out.logits if hasattr(out, "logits") else out
    ours = torch.load("ours_logits.pt")
    torch.testing.assert_close(logits.detach().float(), ours.float(), rtol=1e-4, atol=1e-4)
    """, tmp_path)


@pytest.mark.parametrize("flatten", [False, True])
def test_reference_loads_checkpoint_written_here(tmp_path, flatten):
    from olmo_core_b200.distributed.checkpoint import save_model_and_optim_state

    model, optim = _ours(0)
    for g in optim.param_groups:
        g["lr"], g["weight_decay"] = 4e-3, 0.07
    ids = torch.randint(0, 512, (2, 16))
    model(ids, labels=ids).loss.backward()
    optim.step()
    save_model_and_optim_state(str(tmp_path / "ckpt"), model, optim, flatten_optimizer_state=flatten)
    torch.save({"params": {n: p.detach().clone() for n, p in model.named_parameters()},
                "exp_avg_sq": {n: optim.state[p]["exp_avg_sq"].clone() for n, p in model.named_parameters()}},
               tmp_path / "full.pt")
    _run_reference(_REF_PRELUDE + f"""
    load_model_and_optim_state("ckpt", model, optim, flatten_optimizer_state={flatten})
    want = torch.load("full.pt")
    assert abs(optim.param_groups[0]["lr"] - 4e-3) < 1e-12 and abs(optim.param_groups[0]["weight_decay"] - 0.07) < 1e-12
    for n, p in model.named_parameters():
        assert torch.equal(p.data, want["params"][n]), n
        assert torch.equal(optim.state[p]["exp_avg_sq"], want["exp_avg_sq"][n]), n
    """, tmp_path)
