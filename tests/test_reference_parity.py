"""
Model parity with the reference implementation itself. A child process whose import path holds ONLY the reference
install (``baseline/_ref`` plus its stand-in dependencies) enumerates every named model size and runs forward passes;
this package must build the same parameters (names, shapes, counts) and, given the reference's weights, produce the
reference's logits. Skipped where the reference is not installed.
"""

import json
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

GENERIC_BUILDERS = ("from_dict", "llama_like", "llama_like_moe", "ngpt_like", "gemma3_like", "qwen3_5_like", "build")
FAMILIES = {"olmo2_30M": dict(n_layers=2), "olmo3_190M": dict(n_layers=4), "llama2_271M": dict(n_layers=2),
            "llama3_1B": dict(n_layers=1), "qwen3_0_6B": dict(n_layers=2), "gemma3_1B": dict(n_layers=6),
            "ngpt_271M": dict(n_layers=2), "olmo2_1B_v2": dict(n_layers=1)}


def _run_reference(code: str, cwd: Path) -> None:
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([str(SHIMS), str(REF)])
    env.pop("RANK", None)
    env.pop("WORLD_SIZE", None)
    proc = subprocess.run([sys.executable, "-c", textwrap.dedent(code)], cwd=str(cwd), env=env, capture_output=True,
                          text=True, timeout=1500)
    assert proc.returncode == 0, proc.stderr[-3000:]


def test_every_named_model_size_has_the_reference_parameters(tmp_path):
    out = tmp_path / "ref_models.json"
    _run_reference(f"""
        import inspect, json, olmo_core
        assert "baseline/_ref" in olmo_core.__file__.replace("\\\\", "/"), olmo_core.__file__
        from olmo_core.nn.transformer import TransformerConfig
        out = {{}}
        for name, fn in inspect.getmembers(TransformerConfig, predicate=inspect.ismethod):
            if name.startswith("_") or name in {GENERIC_BUILDERS!r} or "vocab_size" not in inspect.signature(fn).parameters:
                continue
            cfg = fn(vocab_size=1024)
            model = cfg.build(init_device="meta")
            out[name] = dict(params={{k: list(v.shape) for k, v in model.state_dict().items()}}, num_params=cfg.num_params,
                             non_embedding=cfg.num_non_embedding_params)
        json.dump(out, open({str(out)!r}, "w"))
    """, tmp_path)
    from olmo_core_b200.nn.transformer import TransformerConfig

    ref = json.loads(out.read_text())
    assert len(ref) >= 50, sorted(ref)
    problems = []
    for name, want in sorted(ref.items()):
        fn = getattr(TransformerConfig, name, None)
        if fn is None:
            problems.append(f"{name}: missing")
            continue
        cfg = fn(vocab_size=1024)
        got = {k: list(v.shape) for k, v in cfg.build(init_device="meta").state_dict().items()}
        if got != want["params"]:
            problems.append(f"{name}: parameters differ ({sorted(set(got) ^ set(want['params']))[:4]})")
        elif (cfg.num_params, cfg.num_non_embedding_params) != (want["num_params"], want["non_embedding"]):
            problems.append(f"{name}: {cfg.num_params} parameters, reference {want['num_params']}")
    assert not problems, problems


def test_reference_weights_give_reference_logits(tmp_path):
    out = tmp_path / "ref_logits.pt"
    _run_reference(f"""
        import torch, olmo_core
        from olmo_core.nn.transformer import TransformerConfig
        torch.manual_seed(0)
        out = {{}}
        for name, kw in {FAMILIES!r}.items():
            model = getattr(TransformerConfig, name)(vocab_size=512, **kw).build(init_device="cpu")
            model.init_weights(device=torch.device("cpu"), max_seq_len=64)
            model.eval()
            ids = torch.randint(0, 512, (2, 48))
            with torch.no_grad():
                logits = model(ids)
            out[name] = dict(state={{k: v.clone() for k, v in model.state_dict().items()}}, ids=ids, logits=logits)
        torch.save(out, {str(out)!r})
    """, tmp_path)
    from olmo_core_b200.nn.transformer import TransformerConfig

    ref = torch.load(out, weights_only=False)
    assert set(ref) == set(FAMILIES)
    for name, r in ref.items():
        model = getattr(TransformerConfig, name)(vocab_size=512, **FAMILIES[name]).build(init_device="cpu")
        model.init_weights(max_seq_len=64, device=torch.device("cpu"))
        model.load_state_dict(r["state"])
        model.eval()
        with torch.no_grad():
            got = model(r["ids"])
        torch.testing.assert_close(got, r["logits"], rtol=1e-4, atol=2e-5, msg=lambda m, name=name: f"{name}: {m}")


def test_reference_weights_give_reference_loss_and_gradients(tmp_path):
    out = tmp_path / "ref_grads.pt"
    _run_reference(f"""
        import torch, olmo_core
        from olmo_core.nn.transformer import TransformerConfig
        torch.manual_seed(1)
        out = {{}}
        for name, kw in (("olmo2_30M", dict(n_layers=2)), ("qwen3_0_6B", dict(n_layers=1)), ("gemma3_1B", dict(n_layers=6))):
            model = getattr(TransformerConfig, name)(vocab_size=512, **kw).build(init_device="cpu")
            model.init_weights(device=torch.device("cpu"), max_seq_len=64)
            ids = torch.randint(0, 512, (2, 32))
            labels = torch.roll(ids, -1, dims=1)
            labels[:, -1] = -100
            res = model(ids, labels=labels, loss_reduction="sum", z_loss_multiplier=1e-4, loss_div_factor=float((labels != -100).sum()))
            res.loss.backward()
            out[name] = dict(kw=kw, state={{k: v.detach().clone() for k, v in model.state_dict().items()}}, ids=ids, labels=labels,
                             loss=res.loss.detach(), ce=res.ce_loss.detach(), z=res.z_loss.detach(),
                             grads={{k: p.grad.clone() for k, p in model.named_parameters()}})
        torch.save(out, {str(out)!r})
    """, tmp_path)
    from olmo_core_b200.nn.transformer import TransformerConfig

    ref = torch.load(out, weights_only=False)
    for name, r in ref.items():
        model = getattr(TransformerConfig, name)(vocab_size=512, **r["kw"]).build(init_device="cpu")
        model.init_weights(max_seq_len=64, device=torch.device("cpu"))
        model.load_state_dict(r["state"])
        res = model(r["ids"], labels=r["labels"], loss_reduction="sum", z_loss_multiplier=1e-4,
                    loss_div_factor=float((r["labels"] != -100).sum()))
        res.loss.backward()
        torch.testing.assert_close(res.ce_loss.detach(), r["ce"], rtol=1e-5, atol=1e-6, msg=lambda m, n=name: f"{n} ce: {m}")
        torch.testing.assert_close(res.z_loss.detach(), r["z"], rtol=1e-4, atol=1e-7, msg=lambda m, n=name: f"{n} z: {m}")
        torch.testing.assert_close(res.loss.detach(), r["loss"], rtol=1e-5, atol=1e-6, msg=lambda m, n=name: f"{n} loss: {m}")
        for pname, p in model.named_parameters():
            torch.testing.assert_close(p.grad, r["grads"][pname], rtol=2e-3, atol=1e-6,
                                       msg=lambda m, n=name, q=pname: f"{n} {q}: {m}")
