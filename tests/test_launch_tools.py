"""Cluster placement helpers and the code-corpus export (CPU only, no network)."""

import gzip
import json

import numpy as np
import pytest

from olmo_core_b200.data.misc.code_fresh_export import (
    CODE_FRESH_LANGUAGES,
    build_documents_and_stats,
    flatten_documents,
    get_export_dir_name,
    write_document_metadata,
    write_memmap,
    write_stats,
)
from olmo_core_b200.exceptions import BeakerInsufficientResourcesError
from olmo_core_b200.launch.reorder_ranks_in_gcp import topology_order
from olmo_core_b200.launch.select_beaker_hosts import HostMetadata, get_hostname_constraints


def test_topology_order_groups_by_block_and_keeps_rank_zero():
    hosts = ["/b2/s1/m1", "/b1/s1/m1", "/b2/s2/m9", "/b1/s1/m2", "/b2/s1/m0", "/b1/s2/m5"]
    order = topology_order(hosts)
    assert order[0] == 0
    # rank 0's sub-block first (its own machine, then m0), then the rest of its block, then block b1 grouped by sub-block
    assert [hosts[r] for r in order] == ["/b2/s1/m1", "/b2/s1/m0", "/b2/s2/m9", "/b1/s1/m1", "/b1/s1/m2", "/b1/s2/m5"]
    with pytest.raises(ValueError):
        topology_order(["/a/b/c", "/a/b/c"])


def _cluster(sizes):
    return {f"{blk}-{i}": HostMetadata(blk, "s", f"m{i}") for blk, n in sizes.items() for i in range(n)}


def test_host_selection_prefers_one_block_and_keeps_units_together():
    meta = _cluster({"A": 10, "B": 4})
    # a block with more free hosts than needed: every task may use the whole block
    tasks = get_hostname_constraints(meta, num_execution_units=2, num_hosts_per_task=4, num_tasks=2)
    assert len(tasks) == 2 and all(sorted(t) == sorted(h for h in meta if h.startswith("A-")) for t in tasks)
    # otherwise whole execution units per block: 6 free in A, 4 in B, units of 4 hosts
    busy = {f"A-{i}" for i in range(4)}
    tasks = get_hostname_constraints(meta, num_execution_units=2, num_hosts_per_task=8, num_tasks=1, occupied_hosts=busy)
    assert len(tasks[0]) == 8
    for start in (0, 4):
        assert len({meta[h].block for h in tasks[0][start:start + 4]}) == 1
    with pytest.raises(BeakerInsufficientResourcesError):
        get_hostname_constraints(meta, num_execution_units=1, num_hosts_per_task=8, num_tasks=1, occupied_hosts=busy)


class _Tok:
    eos_token_id = 7

    def encode(self, text, add_special_tokens=False):
        return [ord(c) % 5 for c in text]


def test_code_export_round_trip(tmp_path):
    rows = [{"file_contents": "  abc \n"}, {"file_contents": "   "}, {"file_contents": "hello"}]
    docs, stats = build_documents_and_stats(rows, _Tok(), language="python")
    assert stats.num_docs == 2 and stats.num_skipped_empty == 1 and stats.total_tokens == 4 + 6
    assert stats.max_doc_tokens_before_eos == 5 and all(d[-1] == 7 for d in docs)
    tokens, offsets = flatten_documents(docs)
    assert offsets == [(0, 4), (4, 10)] and tokens.dtype == np.uint32
    write_memmap(tmp_path / "x" / "tokens.npy", tokens)
    write_document_metadata(tmp_path / "x" / "tokens.csv.gz", offsets)
    write_stats(tmp_path / "x" / "stats.json", stats)
    assert np.array_equal(np.memmap(tmp_path / "x" / "tokens.npy", dtype=np.uint32, mode="r"), tokens)
    assert gzip.open(tmp_path / "x" / "tokens.csv.gz", "rt").read() == "0,4\n4,10\n"
    assert json.loads((tmp_path / "x" / "stats.json").read_text())["language"] == "python"
    assert not list((tmp_path / "x").glob("*.tmp"))
    with pytest.raises(ValueError):
        build_documents_and_stats([{"file_contents": "x" * 20}], _Tok(), language="c", max_doc_tokens_before_eos=10)
    assert "python" in CODE_FRESH_LANGUAGES and get_export_dir_name("allenai/dolma2-tokenizer").endswith("dolma2-tokenizer")


def test_reshard_checkpoint_script(tmp_path):
    """Two shards in, three shards out (uneven split), same tensors."""
    import torch

    from olmo_core_b200.distributed.checkpoint import get_checkpoint_metadata, load_keys, save_state_dict
    from olmo_core_b200.scripts.reshard_checkpoint import reshard

    state = {"model": {"w": torch.arange(70.0).view(10, 7), "b": torch.ones(3)}, "optim": {"state.w.step": torch.tensor(5.0)}}
    save_state_dict(str(tmp_path / "src"), state)
    reshard(str(tmp_path / "src"), str(tmp_path / "dst"), ranks=3)
    files = sorted(p.name for p in (tmp_path / "dst").iterdir() if p.name.endswith(".distcp"))
    assert {f.split("_")[2] for f in files} == {"0", "1", "2"}
    w, b, step = load_keys(str(tmp_path / "dst"), ["model.w", "model.b", "optim.state.w.step"])
    assert torch.equal(w, state["model"]["w"]) and torch.equal(b, state["model"]["b"]) and float(step) == 5.0
    assert set(get_checkpoint_metadata(str(tmp_path / "dst")).state_dict_metadata) == {"model.w", "model.b", "optim.state.w.step"}
    reshard(str(tmp_path / "src"), str(tmp_path / "dst2"), ranks=2, skip_optimizer_state=True)
    assert set(get_checkpoint_metadata(str(tmp_path / "dst2")).state_dict_metadata) == {"model.w", "model.b"}


def test_compare_wandb_configs_on_local_files(tmp_path, capsys):
    import json

    from olmo_core_b200.scripts import compare_wandb_configs as cw

    assert cw.run_path("https://wandb.ai/ai2/proj/runs/abc123?x=1") == "ai2/proj/abc123" and cw.run_path("a/b/c") == "a/b/c"
    (tmp_path / "l.json").write_text(json.dumps({"model": {"d_model": 128, "n_layers": 2}, "seed": 1}))
    (tmp_path / "r.json").write_text(json.dumps({"model": {"d_model": 256, "n_layers": 2}, "lr": 0.1}))
    cw.main([str(tmp_path / "l.json"), str(tmp_path / "r.json")])
    out = capsys.readouterr().out
    assert "model.d_model: 128 -> 256" in out and "seed = 1" in out and "lr = 0.1" in out and "n_layers" not in out


def test_healthcheck_reads_gpu_state_from_a_fake_nvidia_smi(monkeypatch):
    from olmo_core_b200.scripts import healthcheck as hc

    def smi_factory(rows, procs=""):
        def smi(args):
            return procs if any("compute-apps" in a for a in args) else rows
        return smi

    healthy = "\n".join(f"{i}, 31, 4, 1965, 1965, Not Active, Not Active, Not Active" for i in range(8))
    rep = hc.Report()
    hc.check_gpus(rep, expect_gpus=8, temp_warn=50, temp_fail=55, max_used_mib=1024, smi=smi_factory(healthy))
    assert rep.ok and not rep.warnings

    rep = hc.Report()
    hc.check_gpus(rep, expect_gpus=8, temp_warn=50, temp_fail=55, max_used_mib=1024,
                  smi=smi_factory(healthy.replace("0, 31", "0, 52").replace("3, 31, 4", "3, 61, 90000")
                                  .replace("5, 31, 4, 1965, 1965", "5, 31, 4, 1965, 1200")
                                  .replace("7, 31, 4, 1965, 1965, Not Active", "7, 31, 4, 1965, 1965, Active"),
                                  procs="4242, python, 80000\n"))
    text = " | ".join(rep.failures)
    assert "GPU 3 is at 61 C" in text and "90000 MiB" in text and "hw_slowdown" in text and "compute process" in text
    assert any("GPU 0 is at 52 C" in w for w in rep.warnings) and any("clock lock" in w for w in rep.warnings)

    rep = hc.Report()
    hc.check_gpus(rep, expect_gpus=8, temp_warn=50, temp_fail=55, max_used_mib=1024,
                  smi=smi_factory("\n".join(healthy.splitlines()[:6])))
    assert any("expected 8 GPUs" in f for f in rep.failures)
    monkeypatch.setenv("OLMO_SKIP_HEALTHCHECKS", "1")
    assert hc.main([]) == 0


def test_slurm_script_rendering(tmp_path):
    from olmo_core_b200.launch.slurm import SlurmLaunchConfig

    cfg = SlurmLaunchConfig(name="olmo2-7b", cmd=["python", "-m", "olmo_core_b200.scripts.train", "OLMo2-7B", "--x=a b"],
                            nodes=4, partition="b200", env={"NCCL_DEBUG": "WARN"}, exclude_nodes=["n13"])
    text = cfg.render()
    assert "#SBATCH --nodes=4" in text and "#SBATCH --gpus-per-node=8" in text and "#SBATCH --partition=b200" in text
    assert "#SBATCH --exclude=n13" in text and "export NCCL_DEBUG=WARN" in text
    assert "olmo_core_b200.scripts.healthcheck --expect-gpus 8" in text
    assert "--nnodes=4 --nproc-per-node=8" in text and "-m olmo_core_b200.scripts.train OLMo2-7B '--x=a b'" in text
    path = tmp_path / "job.sbatch"
    assert cfg.launch(str(path), dry_run=True) is None and path.read_text() == text
    import pytest

    with pytest.raises(Exception):
        SlurmLaunchConfig(name="x", cmd=[])


def test_every_training_recipe_builds_a_config():
    """All named recipes assemble into an experiment config on a machine without GPUs or a scheduler."""
    from olmo_core_b200.internal.experiment import CliContext, SubCmd
    from olmo_core_b200.optim import LinearWithWarmup
    from olmo_core_b200.optim.scheduler import WSD
    from olmo_core_b200.scripts.train.recipes import RECIPES, config_builder_for

    assert {"OLMo2-7B-long-context", "OLMo2-7B-anneal", "OLMo3-190M", "OLMo3-7B-anneal", "OLMo-hybrid-7B-long-context",
            "OLMo3-7B-SFT", "OLMoE2-medium", "OLMoE2-large"} <= set(RECIPES)
    for name, recipe in RECIPES.items():
        ctx = CliContext(script="train.py", cmd=SubCmd.dry_run, run_name=f"test-{name}", cluster="local", overrides=[])
        config = config_builder_for(name)(ctx)
        tm = config.train_module
        assert config.model.n_layers > 0 and tm.max_sequence_length == recipe.sequence_length, name
        assert config.data_loader.global_batch_size == recipe.global_batch_sequences * recipe.sequence_length, name
        if recipe.schedule == "decay":
            assert isinstance(tm.scheduler, WSD), name
        if recipe.schedule == "linear":
            assert isinstance(tm.scheduler, LinearWithWarmup), name
        if recipe.cp_degree:
            assert tm.cp_config is not None and tm.cp_config.degree == recipe.cp_degree, name
        if recipe.packed_documents:
            assert config.dataset.label_mask_paths and tm.z_loss_multiplier is None, name
        if recipe.hybrid:
            assert config.model.block_pattern == ["gdn", "gdn", "gdn", "attn"], name
    hybrid_lc = config_builder_for("OLMo-hybrid-7B-long-context")(
        CliContext(script="train.py", cmd=SubCmd.dry_run, run_name="lc", cluster="local", overrides=[]))
    attn = hybrid_lc.model.block["attn"]
    assert (attn.sequence_mixer if getattr(attn, "sequence_mixer", None) is not None else attn.attention).rope is None
    small = config_builder_for("OLMo3-190M")(
        CliContext(script="train.py", cmd=SubCmd.dry_run, run_name="s", cluster="local", overrides=[]))
    assert 2e9 < small.trainer.max_duration.value < 6e9  # 20 tokens per (non-embedding) parameter
