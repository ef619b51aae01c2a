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


SCHEDULER_SPECS = [
    "ConstantScheduler()",
    "ConstantWithWarmup(warmup=10)",
    "ConstantWithWarmup(warmup_fraction=0.1, warmup_min_lr=1e-5)",
    "WSD(warmup=10, decay=20, decay_fraction=None)",
    "WSD(warmup_fraction=0.05, decay_fraction=0.2, decay_min_lr=1e-5)",
    "PowerLR(warmup=10)",
    "PowerLR(warmup=7, b=-0.4, decay=15, decay_fraction=None, decay_min_lr=1e-6)",
    "LinearWithWarmup(warmup=10)",
    "LinearWithWarmup(warmup=5, alpha_f=0.0, t_max=80)",
    "InvSqrtWithWarmup(warmup=12)",
    "InvSqrtWithWarmup(warmup=12, alpha_f=0.3, warmup_min_lr=1e-4)",
    "CosWithWarmup(warmup=10)",
    "CosWithWarmup(warmup_fraction=0.1, alpha_f=0.01, t_max=150)",
    "HalfCosWithWarmup(warmup=10)",
    "CosWithWarmupAndLinearDecay(warmup=10, decay=10, decay_fraction=None)",
    "CosWithWarmupAndLinearDecay(warmup=4, alpha_f=0.2, decay_fraction=0.25, decay_min_lr=1e-5)",
    "ExponentialScheduler()",
    "ExponentialScheduler(lr_min=1e-6)",
    "WSDS(period_lengths=[40, 60], warmup=5, decay=10)",
    "WSDS(period_lengths=[30, 30, 40], period_lr_multipliers=[1.0, 0.5, 0.25], warmup_fraction=0.1, decay_fraction=0.2, decay_min_lr=1e-5)",
    "SequentialScheduler(schedulers=[LinearWithWarmup(warmup=10, alpha_f=0.5), CosWithWarmup(warmup=0)], schedulers_max=[50])",
    "ComposableScheduler(stages=[ComposableSchedulerStage(duration=10, shape='linear', start_lr_fraction=0.0, end_lr_fraction=1.0),"
    " ComposableSchedulerStage(duration=50, shape='cosine', end_lr_fraction=0.1), ComposableSchedulerStage(duration=40, shape='linear', end_lr_fraction=0.0)])",
    "ComposableScheduler(stages=[ComposableSchedulerStage(duration=100, shape='linear', end_lr_fraction=0.5)],"
    " override_decay=OverrideDecay(start=60, duration=20, shape='cosine', end_lr_fraction=0.01))",
]


def _schedule_values(module, specs):
    out = {}
    for spec in specs:
        sched = eval(spec, vars(module))  # noqa: S307 - fixed strings above
        out[spec] = [float(sched.get_lr(3e-4, t, 100)) for t in range(0, 101)]
    return out


def test_learning_rate_schedules_match_the_reference(tmp_path):
    out = tmp_path / "ref_sched.json"
    _run_reference(f"""
        import json
        import olmo_core.optim.scheduler as module
        out = {{}}
        for spec in {SCHEDULER_SPECS!r}:
            sched = eval(spec, vars(module))
            out[spec] = [float(sched.get_lr(3e-4, t, 100)) for t in range(0, 101)]
        json.dump(out, open({str(out)!r}, "w"))
    """, tmp_path)
    import olmo_core_b200.optim.scheduler as module

    want = json.loads(out.read_text())
    got = _schedule_values(module, SCHEDULER_SPECS)
    for spec in SCHEDULER_SPECS:
        assert got[spec] == pytest.approx(want[spec], rel=1e-9, abs=1e-15), spec


def test_data_loader_order_matches_the_reference(tmp_path):
    import numpy as np

    rng = np.random.default_rng(0)
    files = []
    for n, name in ((32 * 40, "a"), (32 * 25 + 7, "b")):
        arr = rng.integers(2, 512, n).astype(np.uint16)
        arr[31::32] = 1
        arr.tofile(tmp_path / f"tokens_{name}.npy")
        files.append(str(tmp_path / f"tokens_{name}.npy"))
    body = """
        import json, os, numpy as np
        def batches(pkg, files, work, out):
            os.makedirs(work, exist_ok=True)
            tok = pkg.TokenizerConfig(vocab_size=512, eos_token_id=1, pad_token_id=0)
            res = {}
            for kind, cls in (("fsl", pkg.NumpyFSLDatasetConfig), ("padded", pkg.NumpyPaddedFSLDatasetConfig)):
                ds = cls(tokenizer=tok, paths=files, sequence_length=32, work_dir=work).build()
                ds.prepare()
                res[kind + "_len"] = len(ds)
                for ws, rank in ((1, 0), (2, 1)):
                    loader = pkg.NumpyFSLDataLoader(ds, collator=pkg.DataCollator(pad_token_id=0), global_batch_size=8 * 32,
                                                    work_dir=work, seed=7, dp_world_size=ws, dp_rank=rank, fs_local_rank=0)
                    loader.reshuffle(epoch=1)
                    seen = []
                    for i, b in enumerate(loader):
                        seen.append(b["input_ids"].tolist())
                        if i == 2:
                            break
                    loader.reset()
                    res[f"{kind}_ws{ws}"] = seen
            json.dump(res, open(out, "w"))
    """
    ref_out, our_out = tmp_path / "ref.json", tmp_path / "ours.json"
    _run_reference(body + f"""
        import olmo_core.data as pkg
        batches(pkg, {files!r}, {str(tmp_path / 'work_ref')!r}, {str(ref_out)!r})
    """, tmp_path)
    namespace = {}
    exec(textwrap.dedent(body), namespace)  # noqa: S102 - the same fixed source the reference ran
    import olmo_core_b200.data as pkg

    namespace["batches"](pkg, files, str(tmp_path / "work_ours"), str(our_out))
    want, got = json.loads(ref_out.read_text()), json.loads(our_out.read_text())
    assert want.keys() == got.keys()
    for key in want:
        assert got[key] == want[key], key


def test_packed_interleaved_and_variable_length_datasets_match_the_reference(tmp_path):
    """Same token files, same seeds: the packed instances (best-fit-decreasing with the reference's tie rules), the woven
    instances of the interleaved dataset, and the variable-length dataset's instances, buckets and batch order."""
    import numpy as np

    rng = np.random.default_rng(1)
    files = []
    for name, n in (("a", 3000), ("b", 2100)):
        arr = rng.integers(2, 512, n).astype(np.uint16)
        pos = 0
        while pos < n:
            pos += int(rng.integers(5, 90))
            if pos < n:
                arr[pos] = 1
        arr[-1] = 1
        arr.tofile(tmp_path / f"tok_{name}.npy")
        files.append(str(tmp_path / f"tok_{name}.npy"))
    body = """
        import json, os, numpy as np
        def dump(pkg, files, work, out):
            os.makedirs(work, exist_ok=True)
            tok = pkg.TokenizerConfig(vocab_size=512, eos_token_id=1, pad_token_id=0)
            res = {}
            ds = pkg.NumpyPackedFSLDatasetConfig(tokenizer=tok, paths=files, sequence_length=64, work_dir=work).build()
            ds.prepare()
            res["packed"] = [np.asarray(ds[i]["input_ids"]).tolist() for i in range(len(ds))]
            ds = pkg.NumpyInterleavedFSLDatasetConfig(tokenizer=tok, paths=files, sequence_length=64, work_dir=work,
                                                      docs_per_instance=2, chunks_per_doc=2, seed=5).build()
            ds.prepare()
            res["interleaved"] = [np.asarray(ds[i]["input_ids"]).tolist() for i in range(len(ds))]
            ds = pkg.NumpyVSLDatasetConfig(tokenizer=tok, paths=files, max_sequence_length=64, min_sequence_length=8, work_dir=work,
                                           vsl_curriculum=pkg.VSLCurriculumConfig(name="grow_p2", num_cycles=2, balanced=False)).build()
            ds.prepare()
            res["vsl"] = [np.asarray(ds[i]["input_ids"]).tolist() for i in range(len(ds))]
            res["vsl_buckets"] = {str(s): np.asarray(ds.get_instance_bucket(s)).tolist() for s, _ in ds.instances_per_bucket}
            per_bucket = ds.curriculum.batches_per_bucket(ds, 128)
            res["vsl_batches_per_bucket"] = [[int(a), int(b)] for a, b in per_bucket]
            res["vsl_batch_order"] = np.asarray(ds.curriculum.get_batch_indices(per_bucket, 4)).tolist()
            json.dump(res, open(out, "w"))
    """
    ref_out, our_out = tmp_path / "ref.json", tmp_path / "ours.json"
    _run_reference(body + f"""
        import olmo_core.data as pkg
        dump(pkg, {files!r}, {str(tmp_path / 'work_ref')!r}, {str(ref_out)!r})
    """, tmp_path)
    namespace = {}
    exec(textwrap.dedent(body), namespace)  # noqa: S102 - the same fixed source the reference ran
    import olmo_core_b200.data as pkg

    namespace["dump"](pkg, files, str(tmp_path / "work_ours"), str(our_out))
    want, got = json.loads(ref_out.read_text()), json.loads(our_out.read_text())
    assert want.keys() == got.keys()
    for key in want:
        assert got[key] == want[key], key


def test_composable_sources_match_the_reference(tmp_path):
    """Token / document / instance sources of the composable data API: concatenation, splits, sampling (down and up),
    mixing, chunking, packing and the global index order give the reference's tokens for the same seeds."""
    body = """
        import json, os, numpy as np
        def dump(C, TokenizerConfig, build_global_indices, work, out):
            os.makedirs(work, exist_ok=True)
            res = {}
            ids = lambda src: np.asarray(src[0:src.num_tokens]["input_ids"]).tolist()
            firsts = lambda src: [np.asarray(src[i]["input_ids"]).tolist()[:2] for i in range(len(src))]
            a = C.InMemoryTokenSource(list(range(100)), work_dir=work, label="a")
            b = C.InMemoryTokenSource(list(range(100, 400)), work_dir=work, label="b")
            res["cat"] = np.asarray((a + b)[95:105]["input_ids"]).tolist()
            res["split"] = [s.num_tokens for s in (a + b).split(0.4)]
            res["resize"] = ids(a.resize(2.5, seed=None))
            res["sample"] = ids(a.sample(max_tokens=10, seed=3))
            res["sample_b"] = ids(b.sample(max_tokens=50, seed=7))
            res["resize_seeded"] = ids(a.resize(1.7, seed=5))
            Spec = C.MixingTokenSource.Spec
            res["mix"] = ids(C.MixingTokenSource(Spec(source=a, ratio=0.5), Spec(source=b, ratio=0.5), work_dir=work, seed=0))
            res["mix_repeat"] = ids(C.MixingTokenSource(Spec(source=a, ratio=0.25, max_repetition_factor=3.0),
                                                        Spec(source=b, ratio=0.75), work_dir=work, seed=2))
            rng = np.random.default_rng(0)
            tokens = []
            for n in rng.integers(2, 9, size=40):
                tokens += list(map(int, rng.integers(5, 50, size=n - 1))) + [0]
            tok = TokenizerConfig(vocab_size=64, eos_token_id=0, pad_token_id=63)
            docs = C.InMemoryDocumentSource(tokens, tokenizer=tok, work_dir=work)
            res["doc_offsets"] = [list(map(int, o)) for o in docs.get_document_offsets()]
            res["docs_half"] = ids(docs.sample_by_docs(max_tokens=len(tokens) // 2, seed=1))
            res["docs_up"] = ids(docs.resize_by_docs(1.5, seed=2))
            DSpec = C.MixingDocumentSource.Spec
            res["doc_mix"] = ids(C.MixingDocumentSource(DSpec(source=docs, ratio=0.5), DSpec(source=docs.sample_by_docs(max_tokens=60, seed=4), ratio=0.5),
                                                        work_dir=work, seed=6))
            chunks = C.ConcatAndChunkInstanceSource(a + b, sequence_length=16, work_dir=work)
            res["chunk"] = [len(chunks), np.asarray(chunks[3]["input_ids"]).tolist()]
            packed = C.PackingInstanceSource(docs, sequence_length=16, work_dir=work, tokenizer=tok)
            res["pack"] = [np.asarray(packed[i]["input_ids"]).tolist() for i in range(len(packed))]
            ia = C.ConcatAndChunkInstanceSource(a, sequence_length=10, work_dir=work)
            ib = C.ConcatAndChunkInstanceSource(b, sequence_length=10, work_dir=work)
            iab = C.ConcatAndChunkInstanceSource(a + b, sequence_length=10, work_dir=work)
            ISpec = C.MixingInstanceSource.Spec
            res["inst_mix"] = firsts(C.MixingInstanceSource(ISpec(source=ia, ratio=0.5), ISpec(source=ib, ratio=0.5), work_dir=work, seed=1))
            res["inst_sample"] = firsts(iab.sample(max_instances=17, seed=4))
            res["inst_resize_up"] = firsts(ia.resize(2.5, seed=9))
            front, back = iab.split(0.3)
            res["inst_split"] = [firsts(front), firsts(back)]
            front, back = iab.split(0.3, seed=11)
            res["inst_split_seeded"] = [firsts(front), firsts(back)]
            # (sampling a source whose max_sequence_length exceeds its sequence_length is left out: the reference writes
            # those sample indices as 64-bit integers and reads them back as 32-bit ones, so every other index is 0)
            rand = C.RandomInstanceSource(tokenizer=tok, sequence_length=16, avg_document_length=6, seed=3, num_instances=6,
                                          max_sequence_length=32, work_dir=work)
            res["random"] = [np.asarray(rand[i]["input_ids"]).tolist() for i in range(len(rand))]
            res["global_indices"] = build_global_indices(40, sequence_length=8, max_sequence_length=32, seed=3).tolist()
            json.dump(res, open(out, "w"), default=int)
    """
    ref_out, our_out = tmp_path / "ref.json", tmp_path / "ours.json"
    _run_reference(body + f"""
        import olmo_core.data.composable as C
        from olmo_core.data import TokenizerConfig
        from olmo_core.data.composable.utils import build_global_indices
        dump(C, TokenizerConfig, build_global_indices, {str(tmp_path / 'work_ref')!r}, {str(ref_out)!r})
    """, tmp_path)
    namespace = {}
    exec(textwrap.dedent(body), namespace)  # noqa: S102 - the same fixed source the reference ran
    import olmo_core_b200.data.composable as C
    from olmo_core_b200.data import TokenizerConfig
    from olmo_core_b200.data.composable.utils import build_global_indices

    namespace["dump"](C, TokenizerConfig, build_global_indices, str(tmp_path / "work_ours"), str(our_out))
    want, got = json.loads(ref_out.read_text()), json.loads(our_out.read_text())
    assert want.keys() == got.keys()
    for key in want:
        assert got[key] == want[key], key


OPTIMIZER_PROGRAM = '''
import json, sys, torch
import {package}.optim as O

def run(cfg, steps, spike_at=None):
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.LayerNorm(32), torch.nn.Linear(32, 8, bias=False))
    opt = cfg.build(model)
    g = torch.Generator().manual_seed(1)
    for s in range(steps):
        x = torch.randn(4, 16, generator=g)
        loss = model(x).pow(2).mean() * (50.0 if s == spike_at else 1.0)
        opt.zero_grad()
        loss.backward()
        if hasattr(opt, "latest_loss"):
            opt.latest_loss = loss.detach()
        opt.step()
    return {{k: v.detach().double().flatten().tolist() for k, v in model.state_dict().items()}}

specs = {{
    "adamw": (lambda: O.AdamWConfig(lr=1e-2, weight_decay=0.1, betas=(0.9, 0.95)), 5, None),
    "adamw_groups": (lambda: O.AdamWConfig(lr=1e-2, weight_decay=0.1, group_overrides=[
        O.OptimGroupOverride(params=["*.bias", "1.*"], opts=dict(weight_decay=0.0))]), 5, None),
    "skip_step_adamw": (lambda: O.SkipStepAdamWConfig(lr=1e-2, weight_decay=0.1, rolling_interval_length=4, sigma_factor=2), 8, 6),
    "lion": (lambda: O.LionConfig(lr=1e-3, weight_decay=0.1), 5, None),
    "skip_step_lion": (lambda: O.SkipStepLionConfig(lr=1e-3, weight_decay=0.1, rolling_interval_length=4, sigma_factor=2), 8, 6),
    "adam": (lambda: O.AdamConfig(lr=1e-2), 5, None),
}}  # Muon / NorMuon / Dion of the reference wrap an external package that is not installed here
out = {{}}
for name, (make, steps, spike) in specs.items():
    out[name] = run(make(), steps, spike)
json.dump(out, open(sys.argv[1], "w"))
'''


def test_optimizers_match_the_reference(tmp_path):
    """A few steps of every optimizer the two packages share, from the same weights and batches (one step of the
    skip-step variants sees a loss spike and must be skipped by both)."""
    ref_out, our_out = tmp_path / "ref_optim.json", tmp_path / "our_optim.json"
    program = tmp_path / "optim_program.py"
    program.write_text(OPTIMIZER_PROGRAM.format(package="olmo_core"))
    _run_reference(f"import runpy, sys; sys.argv = ['x', {str(ref_out)!r}]; runpy.run_path({str(program)!r}, run_name='__main__')",
                   tmp_path)
    program.write_text(OPTIMIZER_PROGRAM.format(package="olmo_core_b200"))
    env = dict(os.environ, PYTHONPATH=str(REPO))
    proc = subprocess.run([sys.executable, str(program), str(our_out)], cwd=str(REPO), env=env, capture_output=True,
                          text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    want, got = json.loads(ref_out.read_text()), json.loads(our_out.read_text())
    assert set(got) == set(want)
    for name in want:
        for key in want[name]:
            # a few fp32 roundings apart (the update is formed in a different order), far below one update (1e-2 to 1e-3)
            assert got[name][key] == pytest.approx(want[name][key], rel=1e-4, abs=2e-6), (name, key)


def _run_both(tmp_path: Path, program: str, stem: str):
    """Run ``program`` (a template with ``{package}``; writes JSON to ``sys.argv[1]``) under the reference and here."""
    ref_out, our_out = tmp_path / f"ref_{stem}.json", tmp_path / f"our_{stem}.json"
    script = tmp_path / f"{stem}_program.py"
    script.write_text(program.format(package="olmo_core"))
    shared = tmp_path / f"{stem}_shared.pt"  # argv[2]: a file the first (reference) run may write for the second
    _run_reference(f"import runpy, sys; sys.argv = ['x', {str(ref_out)!r}, {str(shared)!r}]; "
                   f"runpy.run_path({str(script)!r}, run_name='__main__')", tmp_path)
    script.write_text(program.format(package="olmo_core_b200"))
    proc = subprocess.run([sys.executable, str(script), str(our_out), str(shared)], cwd=str(REPO),
                          env=dict(os.environ, PYTHONPATH=str(REPO)), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    return json.loads(ref_out.read_text()), json.loads(our_out.read_text())


ROPE_PROGRAM = '''
import json, sys, torch
import {package}.nn.rope as R
from {package}.nn.buffer_cache import BufferCache

specs = {{
    "default": lambda: R.RoPEConfig(name="default", theta=10000),
    "default_full_precision": lambda: R.RoPEConfig(name="default", theta=500000, full_precision=True),
    "abf": lambda: R.RoPEConfig(name="default", theta=10000, scaling=R.ABFRoPEScalingConfig(new_theta=500000)),
    "position_interpolation": lambda: R.RoPEConfig(name="default", theta=10000, scaling=R.PIRoPEScalingConfig(factor=2.0)),
    "stepwise": lambda: R.RoPEConfig(name="default", theta=500000, scaling=R.StepwiseRoPEScalingConfig()),
    "yarn": lambda: R.RoPEConfig(name="default", theta=500000, scaling=R.YaRNRoPEScalingConfig(factor=8.0, old_context_len=64)),
    "complex": lambda: R.RoPEConfig(name="complex", theta=10000),
}}
g = torch.Generator().manual_seed(0)
q, k = torch.randn(2, 48, 4, 32, generator=g), torch.randn(2, 48, 2, 32, generator=g)
out = {{}}
for name, make in specs.items():
    rope = make().build(head_size=32, cache=BufferCache())
    qo, ko = rope(q.clone(), k.clone(), head_first=False)
    out[name] = [qo.double().flatten().tolist(), ko.double().flatten().tolist()]
json.dump(out, open(sys.argv[1], "w"))
'''


def test_rotary_embeddings_match_the_reference(tmp_path):
    want, got = _run_both(tmp_path, ROPE_PROGRAM, "rope")
    assert set(got) == set(want)
    for name in want:
        for a, b in zip(got[name], want[name]):
            assert a == pytest.approx(b, rel=1e-5, abs=1e-6), name


INIT_PROGRAM = '''
import json, sys, torch
from {package}.nn.transformer import TransformerConfig

out = {{}}
for name, kw in (("olmo2_30M", dict(n_layers=2)), ("llama2_271M", dict(n_layers=2)), ("qwen3_0_6B", dict(n_layers=1)),
                 ("gemma3_1B", dict(n_layers=2)), ("ngpt_271M", dict(n_layers=2)), ("olmo3_190M", dict(n_layers=2))):
    torch.manual_seed(0)
    model = getattr(TransformerConfig, name)(vocab_size=512, **kw).build(init_device="meta")
    model.init_weights(max_seq_len=64, device=torch.device("cpu"))
    out[name] = {{k: [float(v.double().sum()), float(v.double().abs().sum())] for k, v in model.state_dict().items()}}
json.dump(out, open(sys.argv[1], "w"))
'''


def test_weight_initialisation_matches_the_reference(tmp_path):
    """Same seed, same parameters: every family draws its weights from the same streams in the same order."""
    want, got = _run_both(tmp_path, INIT_PROGRAM, "init")
    for name in want:
        assert set(got[name]) == set(want[name]), name
        for key, sums in want[name].items():
            assert got[name][key] == pytest.approx(sums, rel=1e-6, abs=1e-6), (name, key)


GENERATION_PROGRAM = '''
import json, os, sys
os.environ["TORCHDYNAMO_DISABLE"] = "1"  # the reference compiles its sampling helpers; no C++ toolchain for that on a CPU box
import torch
from {package}.nn.transformer import TransformerConfig
from {package}.generate.generation_module.transformer.generation_module import TransformerGenerationModule
from {package}.generate.generation_module.config import GenerationConfig

torch.manual_seed(0)
model = TransformerConfig.olmo2_30M(vocab_size=512, n_layers=2).build(init_device="cpu")
model.init_weights(max_seq_len=128, device=torch.device("cpu"))
if os.path.exists(sys.argv[2]):
    model.load_state_dict(torch.load(sys.argv[2]))
else:
    torch.save(model.state_dict(), sys.argv[2])
ids = torch.randint(2, 512, (3, 10), generator=torch.Generator().manual_seed(5))
mask = torch.ones_like(ids, dtype=torch.bool)
mask[1, :4] = False  # a left-padded prompt
ids[1, :4] = 0
out = {{}}
# the reference's key / value cache needs a flash-attention backend; its uncached decoding is the oracle for both forms here
for use_cache in ((False,) if "{package}" == "olmo_core" else (True, False)):
    config = GenerationConfig(pad_token_id=0, eos_token_id=1, max_new_tokens=12, use_cache=use_cache, do_sample=False)
    module = TransformerGenerationModule(model, config, device=torch.device("cpu"))
    tokens, _, logprobs = module.generate_batch(ids, attention_mask=mask, return_logprobs=True, completions_only=True,
                                                log_timing=False)
    out[str(use_cache)] = dict(tokens=tokens.tolist(), logprobs=logprobs.double().tolist())
    alone = ids[1:2, 4:]  # the padded row's prompt without its padding
    tokens, _, _ = module.generate_batch(alone, attention_mask=torch.ones_like(alone, dtype=torch.bool),
                                         completions_only=True, log_timing=False)
    out[str(use_cache)]["unpadded_row"] = tokens[0].tolist()
json.dump(out, open(sys.argv[1], "w"))
'''


def test_greedy_generation_matches_the_reference(tmp_path):
    """
    Same weights, a batch whose middle row is a left-padded prompt. Decoding without the key / value cache gives the
    reference's completions and log-probabilities for every row (neither implementation hides the padding from
    attention in that form). Decoding with the cache agrees on the unpadded rows and, for the padded row, gives what
    its prompt gives when decoded alone: the cache's left-pad offsets keep padding out of attention and positions.
    """
    want, got = _run_both(tmp_path, GENERATION_PROGRAM, "generation")
    oracle = want["False"]
    assert got["False"]["tokens"] == oracle["tokens"]
    for a, b in zip(got["False"]["logprobs"], oracle["logprobs"]):
        assert a == pytest.approx(b, rel=1e-3, abs=1e-4)
    for row in (0, 2):
        assert got["True"]["tokens"][row] == oracle["tokens"][row]
        assert got["True"]["logprobs"][row] == pytest.approx(oracle["logprobs"][row], rel=1e-3, abs=1e-4)
    assert got["True"]["tokens"][1] == got["True"]["unpadded_row"] == got["False"]["unpadded_row"] == oracle["unpadded_row"]


TRAIN_MODULE_PROGRAM = '''
import json, os, sys
os.environ["TORCHDYNAMO_DISABLE"] = "1"
import torch
from {package}.nn.transformer import TransformerConfig
from {package}.optim import CosWithWarmup, OptimGroupOverride, SkipStepAdamWConfig
from {package}.train.train_module import TransformerTrainModule


class StubTrainer:
    """What a train module asks of its trainer during a step."""

    def __init__(self, global_batch_size, max_steps):
        self.device = torch.device("cpu")
        self.global_batch_size = global_batch_size
        self.dp_process_group = None
        self.global_step, self.max_steps = 0, max_steps
        self.metrics = {{}}

    def record_metric(self, name, value, reduce_type=None, namespace=None, **kwargs):
        key = name if namespace is None else namespace + "/" + name
        self.metrics.setdefault(key, []).append(float(value))

    def record_ce_loss(self, value, reduce_type=None):
        self.record_metric("ce", value)


SEQ, VOCAB, STEPS = 32, 256, 5
torch.manual_seed(0)
model = TransformerConfig.olmo2_30M(vocab_size=VOCAB, n_layers=2).build(init_device="cpu")
model.init_weights(max_seq_len=SEQ, device=torch.device("cpu"))
if os.path.exists(sys.argv[2]):
    model.load_state_dict(torch.load(sys.argv[2]))
else:
    torch.save(model.state_dict(), sys.argv[2])
model.init_weights = lambda *a, **k: None  # keep these weights when the train module prepares the model
module = TransformerTrainModule(
    model=model,
    optim=SkipStepAdamWConfig(lr=2e-3, weight_decay=0.1, betas=(0.9, 0.95),
                              group_overrides=[OptimGroupOverride(params=["embeddings.weight"], opts=dict(weight_decay=0.0))]),
    rank_microbatch_size=2 * SEQ, max_sequence_length=SEQ, scheduler=CosWithWarmup(warmup=2), max_grad_norm=0.5,
    z_loss_multiplier=1e-4, device=torch.device("cpu"))
trainer = StubTrainer(global_batch_size=4 * SEQ, max_steps=STEPS)
module._attach_trainer(trainer)
g = torch.Generator().manual_seed(9)
for step in range(1, STEPS + 1):
    trainer.global_step = step
    ids = torch.randint(0, VOCAB, (4, SEQ), generator=g)  # two micro-batches of two sequences
    module.zero_grads()
    module.train_batch({{"input_ids": ids}})
    module.optim_step()
keep = ("ce", "train/CE loss", "optim/total grad norm", "optim/LR (group 0)", "optim/LR (group 1)", "train/Z loss")
json.dump(dict(metrics={{k: v for k, v in trainer.metrics.items() if k in keep}},
               weights={{k: [float(v.double().sum()), float(v.double().abs().sum())] for k, v in module.model.state_dict().items()}}),
          open(sys.argv[1], "w"))
'''


def test_training_steps_match_the_reference(tmp_path):
    """Five optimizer steps of the transformer train module on CPU from the same weights and batches: micro-batching,
    loss normalisation, z-loss, gradient clipping, the learning-rate schedule, weight-decay groups and SkipStepAdamW
    leave the same metrics and the same weights behind."""
    want, got = _run_both(tmp_path, TRAIN_MODULE_PROGRAM, "train_module")
    assert want["metrics"], "the reference recorded no metrics"
    for key, values in want["metrics"].items():
        assert key in got["metrics"], (key, sorted(got["metrics"]))
        assert got["metrics"][key] == pytest.approx(values, rel=2e-4, abs=1e-7), key
    for key, (total, magnitude) in want["weights"].items():
        got_total, got_magnitude = got["weights"][key]
        assert got_magnitude == pytest.approx(magnitude, rel=1e-5), key
        assert abs(got_total - total) <= 1e-6 * magnitude + 1e-7, key  # the plain sum cancels: judge it by the magnitude


SOURCE_MIXTURE_PROGRAM = '''
import json, sys
from pathlib import Path
import numpy as np
from {package}.data.source_mixture import SourceMixtureConfig, SourceMixtureDatasetConfig, SourceMixtureList

root = Path(sys.argv[2] + ".data")
root.mkdir(exist_ok=True)
sizes = {{"web": [300_000, 250_000], "code": [120_000], "math": [60_000, 40_000, 30_000]}}
paths = {{}}
for name, counts in sizes.items():
    paths[name] = []
    for i, n in enumerate(counts):
        p = root / (name + "-" + str(i) + ".npy")
        if not p.exists():
            np.random.default_rng(len(name) * 10 + i).integers(0, 1000, n, dtype=np.uint32).tofile(p)
        paths[name].append(str(p))
out = {{}}
for label, ratios, extra in (
    ("plain", dict(web=0.6, code=0.25, math=0.15), dict()),
    ("repeat_small", dict(web=0.4, code=0.2, math=0.4), dict(math=dict(max_repetition_ratio=3.0))),
    ("partial_source", dict(web=0.7, code=0.3), dict(web=dict(max_source_fraction=0.6))),
):
    sources = SourceMixtureList([SourceMixtureConfig(source_name=n, target_ratio=r, paths=paths[n], **extra.get(n, {{}}))
                                 for n, r in ratios.items()])
    config = SourceMixtureDatasetConfig(source_list=sources, requested_tokens=400_000, global_batch_size=64 * 256, seed=7,
                                        quiet=True, render_tables=False)
    config.validate()
    mixture = config.build(npdtype=np.uint32, sequence_length=256)
    out[label] = {{Path(p).name + ":" + str(i): int(t) for (p, i), t in mixture.to_index().items()}}
json.dump(out, open(sys.argv[1], "w"))
'''


def test_source_mixtures_match_the_reference(tmp_path):
    """Token budgets per file of a sampled source mixture (plain ratios, a small source that is repeated, a source that
    may only be used in part) come out as in the reference."""
    want, got = _run_both(tmp_path, SOURCE_MIXTURE_PROGRAM, "source_mixture")
    assert got == want


HF_STATE_PROGRAM = '''
import json, sys, torch
from {package}.nn.hf.config import get_hf_config
from {package}.nn.hf.convert import convert_state_from_hf, convert_state_to_hf
from {package}.nn.transformer import TransformerConfig

out = {{}}
for name, kw in (("olmo2_30M", dict(n_layers=2)), ("olmo3_190M", dict(n_layers=4)), ("gemma3_1B", dict(n_layers=6))):
    torch.manual_seed(0)
    model = getattr(TransformerConfig, name)(vocab_size=512, **kw).build(init_device="cpu")
    model.init_weights(max_seq_len=64, device=torch.device("cpu"))
    try:
        hf_config = get_hf_config(model)
    except NotImplementedError as e:
        out[name] = "not exportable: " + str(e)[:60]
        continue
    state = {{k: v.detach().clone() for k, v in model.state_dict().items()}}
    hf_state = convert_state_to_hf(hf_config, state)
    back = convert_state_from_hf(hf_config, {{k: v.clone() for k, v in hf_state.items()}}, model_type=hf_config.model_type)
    out[name] = dict(
        model_type=hf_config.model_type,
        hf={{k: [list(v.shape), float(v.double().sum()), float(v.double().abs().sum())] for k, v in hf_state.items()}},
        round_trip=sorted(k for k in state if k in back and torch.equal(back[k], state[k])),
        config={{k: v for k, v in hf_config.to_dict().items()
                 if k in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                          "rope_theta", "rms_norm_eps", "vocab_size", "sliding_window", "layer_types", "head_dim",
                          "tie_word_embeddings", "max_position_embeddings")}})
json.dump(out, open(sys.argv[1], "w"))
'''


def test_hugging_face_state_conversion_matches_the_reference(tmp_path):
    """The Hugging Face config that is derived from a model, the converted state dict (names, shapes, values) and the way
    back are those of the reference, for every family the reference can export."""
    want, got = _run_both(tmp_path, HF_STATE_PROGRAM, "hf_state")
    exportable = [name for name, value in want.items() if isinstance(value, dict)]
    assert exportable, want
    for name in exportable:
        assert isinstance(got[name], dict), (name, got[name])
        assert got[name]["model_type"] == want[name]["model_type"], name
        assert got[name]["config"] == want[name]["config"], name
        assert set(got[name]["hf"]) == set(want[name]["hf"]), name
        for key, (shape, total, magnitude) in want[name]["hf"].items():
            g_shape, g_total, g_magnitude = got[name]["hf"][key]
            assert g_shape == shape and g_magnitude == pytest.approx(magnitude, rel=1e-6), (name, key)
            assert abs(g_total - total) <= 1e-6 * magnitude + 1e-9, (name, key)
        assert got[name]["round_trip"] == want[name]["round_trip"], name


HF_IMPORT_PROGRAM = '''
import json, sys, torch, transformers
from {package}.nn.hf.convert import convert_state_from_hf

common = dict(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, max_position_embeddings=64)
configs = {{
    "llama": transformers.LlamaConfig(**common),
    "qwen3": transformers.Qwen3Config(head_dim=16, **common),
    "olmo2": transformers.Olmo2Config(**common),
    "olmo3": transformers.Olmo3Config(sliding_window=16, **common),
    "gemma3_text": transformers.Gemma3TextConfig(head_dim=16, sliding_window=16, **common),
}}
out = {{}}
for name, config in configs.items():
    torch.manual_seed(1)
    hf_state = transformers.AutoModelForCausalLM.from_config(config).state_dict()
    try:
        state = convert_state_from_hf(config, {{k: v.clone() for k, v in hf_state.items()}}, model_type=config.model_type)
    except Exception as e:
        out[name] = "error: " + type(e).__name__
        continue
    out[name] = {{k: [list(v.shape), float(v.double().sum()), float(v.double().abs().sum())] for k, v in state.items()}}
json.dump(out, open(sys.argv[1], "w"))
'''


def test_hugging_face_state_import_matches_the_reference(tmp_path):
    """Hugging Face checkpoints of five architectures (random weights from one seed) convert to the same parameter names,
    shapes and values as with the reference."""
    want, got = _run_both(tmp_path, HF_IMPORT_PROGRAM, "hf_import")
    converted = [name for name, value in want.items() if isinstance(value, dict)]
    assert len(converted) >= 3, want
    for name in converted:
        assert isinstance(got[name], dict), (name, got[name])
        assert set(got[name]) == set(want[name]), (name, sorted(set(got[name]) ^ set(want[name])))
        for key, (shape, total, magnitude) in want[name].items():
            g_shape, g_total, g_magnitude = got[name][key]
            assert g_shape == shape and g_magnitude == pytest.approx(magnitude, rel=1e-6), (name, key)
            assert abs(g_total - total) <= 1e-6 * magnitude + 1e-9, (name, key)


ROUTER_PROGRAM = '''
import json, sys, torch
from {package}.nn.moe import MoERouterConfig
from {package}.nn.moe.router import MoERouterGatingFunction

out = {{}}
x = torch.randn(2, 24, 32, generator=torch.Generator().manual_seed(0))
variants = {{
    "softmax_top2": dict(top_k=2),
    "softmax_top4_normalised": dict(top_k=4, normalize_expert_weights=1.0),
    "sigmoid_top2": dict(top_k=2, gating_function=MoERouterGatingFunction.sigmoid),
    "uniform_assignment": dict(top_k=2, uniform_expert_assignment=True),
    "bias_balanced": dict(top_k=2, bias_gamma=0.01),
}}
for name, kw in variants.items():
    torch.manual_seed(1)
    router = MoERouterConfig(**kw).build(32, 8, lb_loss_weight=0.01, z_loss_weight=0.001, init_device="cpu")
    with torch.no_grad():
        for p in router.parameters():
            p.copy_(torch.randn(p.shape, generator=torch.Generator().manual_seed(2)) * 0.5)
    router.train()
    xin = x.clone().requires_grad_(True)
    weights, indices, counts, aux = router(xin, loss_div_factor=48.0)
    total = weights.sum() * 0.1 + (aux if aux is not None else 0.0)
    total.backward()
    order = torch.argsort(indices, dim=-1)  # top-k order within a token is an implementation detail
    out[name] = dict(indices=torch.gather(indices, -1, order).tolist(),
                     weights=torch.gather(weights.detach(), -1, order).double().tolist(),
                     counts=counts.tolist(), aux=None if aux is None else float(aux),
                     dx=[float(xin.grad.double().sum()), float(xin.grad.double().abs().sum())],
                     dw=[float(router.weight.grad.double().abs().sum())],
                     metrics={{k: float(v[0]) for k, v in router.compute_metrics(reset=True).items()}})
json.dump(out, open(sys.argv[1], "w"))
'''


def test_moe_router_matches_the_reference(tmp_path):
    """Expert choice, routing weights, token counts, the auxiliary losses with their gradients and the logged statistics
    of the router, for five gating variants."""
    want, got = _run_both(tmp_path, ROUTER_PROGRAM, "router")
    for name in want:
        w, g = want[name], got[name]
        assert g["indices"] == w["indices"] and g["counts"] == w["counts"], name
        assert g["aux"] == pytest.approx(w["aux"], rel=1e-5), name
        for key in ("dx", "dw"):
            assert g[key] == pytest.approx(w[key], rel=1e-4, abs=1e-7), (name, key)
        for a, b in zip(g["weights"], w["weights"]):
            for row_a, row_b in zip(a, b):
                assert row_a == pytest.approx(row_b, rel=1e-5, abs=1e-7), name
        assert set(g["metrics"]) == set(w["metrics"]), (name, sorted(set(g["metrics"]) ^ set(w["metrics"])))
        for key, value in w["metrics"].items():
            assert g["metrics"][key] == pytest.approx(value, rel=1e-5, abs=1e-8), (name, key)


BATCH_UTILS_PROGRAM = '''
import json, sys, torch
from {package}.data import DataCollator
from {package}.data.utils import get_cumulative_document_lengths, get_document_lengths, get_labels, melt_batch, split_batch, truncate_batch

g = torch.Generator().manual_seed(0)
items = []
for n in (16, 11, 16, 7):
    ids = torch.randint(2, 50, (n,), generator=g)
    ids[n // 2] = 1  # an end-of-document token
    items.append(dict(input_ids=ids, label_mask=torch.rand(n, generator=g) > 0.2, doc_lens=torch.tensor([n // 2 + 1, n - n // 2 - 1]),
                      max_doc_lens=[max(n // 2 + 1, n - n // 2 - 1)], metadata=dict(path="p", index=n)))
batch = DataCollator(pad_token_id=0)(items)
out = {{}}
def dump(prefix, b):
    for k, v in b.items():
        out[prefix + "/" + k] = v.tolist() if torch.is_tensor(v) else (v if isinstance(v, (list, int, float, str)) else str(v))
dump("collated", batch)
out["labels"] = get_labels(batch).tolist()
for i, part in enumerate(split_batch({{k: v for k, v in batch.items() if k != "metadata"}}, 2)):
    dump("split" + str(i), part)
full = dict(input_ids=torch.arange(64).view(2, 32), label_mask=torch.ones(2, 32, dtype=torch.bool))
dump("melted", melt_batch(full, 8))
dump("truncated", truncate_batch(full, 8))
lens = get_document_lengths(torch.tensor([5, 1, 7, 8, 1, 9, 9, 9]), eos_token_id=1)
out["doc_lens"] = lens.tolist()
out["cu_doc_lens"] = get_cumulative_document_lengths(torch.tensor([[3, 5, 0], [4, 4, 0]])).tolist()
json.dump(out, open(sys.argv[1], "w"))
'''


def test_batch_utilities_match_the_reference(tmp_path):
    """Collation with left/right padding, document lengths and masks; label shifting; splitting into micro-batches;
    melting / truncating to a shorter sequence length; document-length helpers."""
    want, got = _run_both(tmp_path, BATCH_UTILS_PROGRAM, "batch_utils")
    assert set(got) == set(want), sorted(set(got) ^ set(want))
    for key in want:
        assert got[key] == want[key], key


ATTENTION_PROGRAM = '''
import json, sys, torch
from {package}.nn.attention import AttentionConfig, AttentionType, GateConfig, GateGranularity
from {package}.nn.layer_norm import LayerNormConfig, LayerNormType
from {package}.nn.rope import RoPEConfig

rms = LayerNormConfig(name=LayerNormType.rms, bias=False)
variants = {{
    "plain": dict(),
    "grouped_query_bias": dict(n_kv_heads=2, bias=True),
    "multi_query_clipped": dict(n_kv_heads=1, clip_qkv=0.4),
    "full_width_qk_norm_rope": dict(qk_norm=rms, rope=RoPEConfig(theta=10000)),
    "per_head_qk_norm_rope": dict(n_kv_heads=2, qk_norm=rms, use_head_qk_norm=True, rope=RoPEConfig(theta=500000)),
    "explicit_head_dim": dict(head_dim=24, rope=RoPEConfig(theta=10000)),
    "headwise_gate": dict(gate=GateConfig(granularity=GateGranularity.headwise)),
    "elementwise_gate": dict(n_kv_heads=2, gate=GateConfig(granularity=GateGranularity.elementwise)),
    "fused_qkv": dict(name=AttentionType.fused),
}}
out = {{}}
x = torch.randn(2, 20, 64, generator=torch.Generator().manual_seed(0))
for name, kw in variants.items():
    try:
        module = AttentionConfig(n_heads=4, **kw).build(64, layer_idx=0, n_layers=2, init_device="cpu")
    except Exception as e:
        out[name] = "build error: " + type(e).__name__
        continue
    g = torch.Generator().manual_seed(3)
    with torch.no_grad():
        for p in module.parameters():
            p.copy_(torch.randn(p.shape, generator=g) * (0.2 if p.dim() > 1 else 1.0))
    xin = x.clone().requires_grad_(True)
    try:
        y = module(xin)
    except Exception as e:
        out[name] = "forward error: " + type(e).__name__
        continue
    (y * torch.linspace(-1, 1, y.numel()).view_as(y)).sum().backward()
    out[name] = dict(params=sorted(k for k, _ in module.named_parameters()), y=y.detach().double().flatten().tolist(),
                     dx=xin.grad.double().flatten().tolist(),
                     dparams={{k: float(p.grad.double().abs().sum()) for k, p in module.named_parameters()}})
json.dump(out, open(sys.argv[1], "w"))
'''


def test_attention_module_variants_match_the_reference(tmp_path):
    """The attention module on CPU for nine option sets (grouped / multi-query, biases, clipping, both QK-norm forms with
    rotary embeddings, explicit head size, both output gates, fused projection): parameter names, outputs, input and
    parameter gradients."""
    want, got = _run_both(tmp_path, ATTENTION_PROGRAM, "attention")
    ran = [name for name, value in want.items() if isinstance(value, dict)]
    assert len(ran) >= 6, want
    for name in ran:
        g, w = got[name], want[name]
        assert isinstance(g, dict), (name, g)
        assert g["params"] == w["params"], name
        assert g["y"] == pytest.approx(w["y"], rel=1e-4, abs=1e-5), name
        assert g["dx"] == pytest.approx(w["dx"], rel=1e-4, abs=1e-5), name
        for key, value in w["dparams"].items():
            # (the key bias has a zero gradient in exact arithmetic: softmax ignores a shift of all scores of a query;
            # what is left there is rounding noise, hence the absolute tolerance)
            assert g["dparams"][key] == pytest.approx(value, rel=1e-4, abs=5e-4), (name, key)


BLOCKS_PROGRAM = '''
import json, sys, torch
from {package}.nn.feed_forward import ActivationFunction, FeedForwardConfig
from {package}.nn.layer_norm import LayerNormConfig, LayerNormType
from {package}.nn.lm_head import LMHeadConfig
from {package}.nn.transformer import TransformerBlockType, TransformerConfig

out = {{}}
x = torch.randn(3, 10, 48, generator=torch.Generator().manual_seed(0))

def fill(module, seed):
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for p in module.parameters():
            p.copy_(torch.randn(p.shape, generator=g) * (0.2 if p.dim() > 1 else 0.5) + (1.0 if p.dim() == 1 else 0.0))

def run(name, module, *args, **kwargs):
    fill(module, 5)
    xin = x.clone().requires_grad_(True)
    y = module(xin, *args, **kwargs)
    y = y if torch.is_tensor(y) else y.loss
    (y.float() * torch.linspace(-1, 1, y.numel()).view_as(y)).sum().backward()
    out[name] = dict(params=sorted(k for k, _ in module.named_parameters()), y=y.detach().double().flatten().tolist(),
                     dx=xin.grad.double().flatten().tolist())

for kind in (LayerNormType.default, LayerNormType.rms, LayerNormType.qwen_rms):
    for kw in (dict(), dict(bias=False), dict(elementwise_affine=False), dict(full_precision=False, eps=1e-3)):
        try:
            run("norm/" + str(kind) + "/" + json.dumps(kw, sort_keys=True), LayerNormConfig(name=kind, **kw).build(48, init_device="cpu"))
        except Exception as e:
            out["norm/" + str(kind) + "/" + json.dumps(kw, sort_keys=True)] = "error: " + type(e).__name__
for act in (ActivationFunction.silu, ActivationFunction.gelu_tanh):
    for bias in (False, True):
        run("mlp/" + str(act) + "/" + str(bias), FeedForwardConfig(hidden_size=96, bias=bias, activation=act).build(48, init_device="cpu"))
labels = torch.randint(0, 64, (3, 10), generator=torch.Generator().manual_seed(1))
labels[0, :2] = -100
for reduction, extra in (("mean", dict()), ("sum", dict(loss_div_factor=9.0, z_loss_multiplier=1e-3)), ("none", dict(z_loss_multiplier=1e-3))):
    head = LMHeadConfig(layer_norm=LayerNormConfig(name=LayerNormType.rms), bias=True).build(d_model=48, vocab_size=64, init_device="cpu")
    run("head/" + reduction, head, labels=labels, loss_reduction=reduction, **extra)
ids = torch.randint(0, 64, (2, 12), generator=torch.Generator().manual_seed(2))
for block in (TransformerBlockType.default, TransformerBlockType.default_scaled, TransformerBlockType.reordered_norm,
              TransformerBlockType.peri_norm):
    model = TransformerConfig.llama_like(d_model=48, vocab_size=64, n_layers=3, n_heads=4, block_name=block).build(init_device="cpu")
    fill(model, 7)
    model.eval()
    with torch.no_grad():
        out["model/" + str(block)] = dict(params=sorted(k for k, _ in model.named_parameters()),
                                          y=model(ids).double().flatten().tolist(), dx=[])
json.dump(out, open(sys.argv[1], "w"))
'''


def test_norms_mlps_heads_and_block_types_match_the_reference(tmp_path):
    """Layer norms (three kinds, with / without affine parameters and bias, low precision), gated MLPs (two activations,
    with bias), the LM head with its three loss reductions, and four block types in a small model."""
    want, got = _run_both(tmp_path, BLOCKS_PROGRAM, "blocks")
    ran = [name for name, value in want.items() if isinstance(value, dict)]
    assert len(ran) >= 15, {k: v for k, v in want.items() if not isinstance(v, dict)}
    for name in ran:
        g, w = got[name], want[name]
        assert isinstance(g, dict), (name, g)
        assert g["params"] == w["params"], name
        assert g["y"] == pytest.approx(w["y"], rel=2e-4, abs=2e-5), name
        assert g["dx"] == pytest.approx(w["dx"], rel=2e-4, abs=2e-5), name


CONFIG_PROGRAM = '''
import json, sys
from {package}.config import DType
from {package}.data import TokenizerConfig
from {package}.nn.transformer import TransformerConfig
from {package}.optim import AdamWConfig, CosWithWarmup, OptimGroupOverride
from {package}.train import Duration
from {package}.train.train_module import TransformerDataParallelConfig, TransformerTrainModuleConfig

out = {{}}
for name in ("dolma2", "gpt_neox_olmo_dolma_v1_5", "gpt2", "llama2", "llama3") if True else ():
    make = getattr(TokenizerConfig, name, None)
    if make is None:
        continue
    tok = make()
    out["tokenizer/" + name] = dict(tok.as_dict(), padded=tok.padded_vocab_size())

def strip(d):
    """Class names differ by package name only."""
    if isinstance(d, dict):
        return {{k: (v.replace("{package}", "PKG") if k == "_CLASS_" else strip(v)) for k, v in d.items()}}
    if isinstance(d, list):
        return [strip(v) for v in d]
    return d

model = TransformerConfig.olmo2_30M(vocab_size=512, n_layers=2)
out["model/as_config_dict"] = strip(model.as_config_dict())
merged = model.merge(["n_layers=5", "block.feed_forward.hidden_size=96", "lm_head.bias=true"])
out["model/merged"] = [merged.n_layers, merged.block.feed_forward.hidden_size, merged.lm_head.bias, model.n_layers]
out["model/round_trip_equal"] = TransformerConfig.from_dict(model.as_config_dict()) == model
out["model/counts"] = [model.num_params, model.num_non_embedding_params, model.num_active_params]
tm = TransformerTrainModuleConfig(
    rank_microbatch_size=1024, max_sequence_length=128, z_loss_multiplier=1e-5, max_grad_norm=1.0,
    optim=AdamWConfig(lr=1e-3, group_overrides=[OptimGroupOverride(params=["embeddings.weight"], opts=dict(weight_decay=0.0))]),
    scheduler=CosWithWarmup(warmup=10),
    dp_config=TransformerDataParallelConfig(name="hsdp", param_dtype=DType.bfloat16, reduce_dtype=DType.float32, shard_degree=4))
out["train_module/as_config_dict"] = strip(tm.as_config_dict())
out["train_module/merged"] = strip(tm.merge(["optim.lr=0.5", "dp_config.shard_degree=8", "scheduler.warmup=3"]).as_config_dict())
out["duration"] = [[d.value, str(d.unit)] for d in (Duration.steps(5), Duration.epochs(2), Duration.tokens(10**9),
                                                  Duration.chinchilla_tokens(2.0, model_params=10**6))]
json.dump(out, open(sys.argv[1], "w"), default=str, sort_keys=True)
'''


def test_config_system_and_value_types_match_the_reference(tmp_path):
    """Tokenizer presets, the serialised form of a model config and of a train-module config, dot-list overrides, the way
    back from a dict, parameter / FLOP counts and durations."""
    want, got = _run_both(tmp_path, CONFIG_PROGRAM, "config")
    assert set(got) == set(want), sorted(set(got) ^ set(want))
    for key in want:
        assert got[key] == want[key], key


LOADER_STATE_PROGRAM = '''
import json, os, sys
import numpy as np
import {package}.data as pkg

root = sys.argv[2] + ".data"
os.makedirs(root, exist_ok=True)
path = os.path.join(root, "tokens.npy")
if not os.path.exists(path):
    arr = np.random.default_rng(0).integers(2, 512, 32 * 64).astype(np.uint16)
    arr[31::32] = 1
    arr.tofile(path)
work = os.path.join(root, "work-{package}")
tok = pkg.TokenizerConfig(vocab_size=512, eos_token_id=1, pad_token_id=0)
ds = pkg.NumpyFSLDatasetConfig(tokenizer=tok, paths=[path], sequence_length=32, work_dir=work).build()
ds.prepare()

def loader(batch=8 * 32):
    return pkg.NumpyFSLDataLoader(ds, collator=pkg.DataCollator(pad_token_id=0), global_batch_size=batch, work_dir=work, seed=3,
                                  dp_world_size=1, dp_rank=0, fs_local_rank=0)

first = loader()
first.reshuffle(epoch=1)
it = iter(first)
seen = [next(it)["input_ids"].tolist() for _ in range(3)]
state = first.state_dict()
rest = [b["input_ids"].tolist() for b in it]
first.reset()
resumed = loader()
resumed.load_state_dict(state)
resumed.reshuffle(epoch=1)
resumed_rest = [b["input_ids"].tolist() for b in resumed]
resumed.reset()
half = loader(batch=4 * 32)  # the batch size halves across the restart: the position in the data is kept
half.load_state_dict(state)
half.reshuffle(epoch=1)
half_rest = [b["input_ids"].tolist() for b in half]
half.reset()
clean = {{k: (v if isinstance(v, (int, float, str, bool, type(None))) else str(type(v).__name__)) for k, v in state.items()
          if k != "dataset_fingerprint"}}
json.dump(dict(state=clean, total=first.total_batches, resumed_equal=resumed_rest == rest, rest=rest, half_rest=half_rest,
               tokens_per_batch=[len(b) * 32 for b in seen]), open(sys.argv[1], "w"), sort_keys=True)
'''


def test_data_loader_state_and_resumption_match_the_reference(tmp_path):
    """The loader's state dict (keys and values), resuming in the middle of an epoch, and resuming with half the batch
    size give the reference's state and the reference's remaining batches."""
    want, got = _run_both(tmp_path, LOADER_STATE_PROGRAM, "loader_state")
    assert want["resumed_equal"] is True and got["resumed_equal"] is True
    for key in want:
        assert got[key] == want[key], key


TRAINER_PROGRAM = '''
import json, os, sys
os.environ["TORCHDYNAMO_DISABLE"] = "1"
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict
import numpy as np
import torch
from {package}.data import DataCollator, NumpyFSLDataLoader, NumpyFSLDatasetConfig, TokenizerConfig
from {package}.nn.transformer import TransformerConfig
from {package}.optim import AdamWConfig, CosWithWarmup
from {package}.train import Duration, TrainerConfig
from {package}.train.callbacks import Callback, CheckpointerCallback
from {package}.train.train_module import TransformerTrainModule

VOCAB, SEQ, STEPS = 512, 32, 6
root = Path(sys.argv[2] + ".data")
root.mkdir(exist_ok=True)
data = root / "tokens.npy"
if not data.exists():
    arr = np.random.default_rng(0).integers(2, VOCAB, 64 * SEQ * 8).astype(np.uint16)
    arr[SEQ - 1:: SEQ] = 1
    arr.tofile(data)


@dataclass
class Recorder(Callback):
    seen: Dict[int, Dict[str, float]] = field(default_factory=dict)

    def log_metrics(self, step, metrics):
        self.seen.setdefault(step, {{}}).update({{k: float(v) for k, v in metrics.items()}})


work = root / "work-{package}"
tok = TokenizerConfig(vocab_size=VOCAB, eos_token_id=1, pad_token_id=0)
ds = NumpyFSLDatasetConfig(tokenizer=tok, paths=[str(data)], sequence_length=SEQ, work_dir=str(work)).build()
ds.prepare()
loader = NumpyFSLDataLoader(ds, collator=DataCollator(pad_token_id=0), global_batch_size=8 * SEQ, work_dir=work, seed=1,
                            dp_world_size=1, dp_rank=0, fs_local_rank=0)
torch.manual_seed(0)
model = TransformerConfig.olmo2_30M(vocab_size=VOCAB, n_layers=2).build(init_device="cpu")
model.init_weights(max_seq_len=SEQ, device=torch.device("cpu"))
if os.path.exists(sys.argv[2]):
    model.load_state_dict(torch.load(sys.argv[2]))
else:
    torch.save(model.state_dict(), sys.argv[2])
model.init_weights = lambda *a, **k: None
module = TransformerTrainModule(model=model, optim=AdamWConfig(lr=1e-3), rank_microbatch_size=2 * SEQ, max_sequence_length=SEQ,
                                scheduler=CosWithWarmup(warmup=2), max_grad_norm=1.0, z_loss_multiplier=1e-5,
                                device=torch.device("cpu"))
rec = Recorder()
run = root / "run-{package}"
config = TrainerConfig(save_folder=str(run), max_duration=Duration.steps(STEPS), metrics_collect_interval=2, save_overwrite=True,
                       device="cpu", cancel_check_interval=1,
                       callbacks={{"rec": rec, "checkpointer": CheckpointerCallback(save_interval=3, save_async=False,
                                                                                    pre_train_checkpoint=False)}})
trainer = config.build(module, loader)
trainer.fit()
keep = ("train/CE loss", "train/Z loss", "train/PPL", "optim/total grad norm", "optim/LR (group 0)")
files = sorted(str(p.relative_to(run)) for p in run.rglob("*") if p.is_file() and "model_and_optim" not in str(p))
shards = sorted(p.name for p in (run / ("step" + str(STEPS)) / "model_and_optim").iterdir())
json.dump(dict(metrics={{str(s): {{k: v for k, v in m.items() if k in keep}} for s, m in rec.seen.items()}},
               metric_names=sorted({{k for m in rec.seen.values() for k in m if not k.startswith(("throughput", "system"))}}),
               files=files, shards=shards, global_step=trainer.global_step, tokens=trainer.global_train_tokens_seen),
          open(sys.argv[1], "w"), sort_keys=True)
'''


def test_a_short_training_run_matches_the_reference(tmp_path):
    """
    ``Trainer.fit`` for six steps on CPU from the same weights and data: the logged metrics (names and values per
    step), the files a run leaves behind (checkpoint folders, trainer state, metadata) and the step / token counters.
    No checkpoint is written before the first step: in the reference that save initialises the optimizer state through
    ``torch.distributed.checkpoint``, which takes one optimizer step with zero gradients and a zero learning rate, so
    that Adam's step counter (and with it the bias correction of the first updates) starts at one instead of zero.
    Weights are untouched by it, and this package does not imitate it.
    """
    want, got = _run_both(tmp_path, TRAINER_PROGRAM, "trainer")
    assert got["global_step"] == want["global_step"] and got["tokens"] == want["tokens"]
    assert got["files"] == want["files"], (sorted(set(got["files"]) ^ set(want["files"])))
    assert got["shards"] == want["shards"]
    assert set(want["metric_names"]) <= set(got["metric_names"]), sorted(set(want["metric_names"]) - set(got["metric_names"]))
    steps = lambda run: {s for s, values in run["metrics"].items() if values}  # noqa: E731  (steps with training metrics)
    assert steps(got) == steps(want) == {str(s) for s in range(1, 7)}
    for step, values in want["metrics"].items():
        for key, value in values.items():
            assert got["metrics"][step][key] == pytest.approx(value, rel=2e-4, abs=1e-7), (step, key)
