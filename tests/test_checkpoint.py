"""Sharded checkpoint format: round trips, resharding across world sizes, unsharding and key utilities (CPU)."""

import pickle

import pytest
import torch
import torch.distributed as dist

from olmo_core_b200.distributed.checkpoint import (
    UnshardStrategy,
    async_save_state_dict,
    get_checkpoint_metadata,
    load_keys,
    load_model_and_optim_state,
    load_state_dict,
    merge_state_dicts,
    prune_state_dict,
    save_model_and_optim_state,
    save_state_dict,
    swap_param_keys,
    unshard_checkpoint,
)
from olmo_core_b200.nn.transformer import TransformerConfig
from olmo_core_b200.optim import AdamWConfig
from olmo_core_b200.testing import run_distributed_test


def _tiny_model(seed: int = 0, sharded: bool = False):
    torch.manual_seed(seed)
    cfg = TransformerConfig.olmo2_30M(vocab_size=512, n_layers=2)
    model = cfg.build(init_device="cpu")
    if sharded:
        model.apply_fsdp(dp_mesh=None, param_dtype=None, reduce_dtype=torch.float32)
        model._sharding_runtime.materialize(torch.device("cpu"))
    model.init_weights(max_seq_len=64, device=torch.device("cpu"))
    if sharded:
        model._sharding_runtime.sync_lowp()
    return model


def _train_a_little(model, optim, steps: int = 2, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    rt = getattr(model, "_sharding_runtime", None)
    for _ in range(steps):
        ids = torch.randint(0, 512, (2, 16), generator=g)
        out = model(ids, labels=ids)
        loss = out.loss if hasattr(out, "loss") else out
        loss.backward()
        if rt is not None:
            rt.reduce_gradients()
        optim.step()
        if rt is not None:
            rt.zero_grad()
        optim.zero_grad(set_to_none=True)


def test_nested_state_dict_round_trip(tmp_path):
    sd = {"a": {"w": torch.arange(12.0).view(3, 4), "n": 7}, "b": torch.ones(5, dtype=torch.bfloat16), "meta": {"x": "y"}}
    save_state_dict(tmp_path / "ckpt", sd)
    files = sorted(p.name for p in (tmp_path / "ckpt").iterdir())
    assert ".metadata" in files and any(f.startswith("__0_") and f.endswith(".distcp") for f in files)
    target = {"a": {"w": torch.zeros(3, 4), "n": 0}, "b": torch.zeros(5, dtype=torch.bfloat16), "meta": {"x": ""}}
    load_state_dict(tmp_path / "ckpt", target)
    assert torch.equal(target["a"]["w"], sd["a"]["w"]) and target["a"]["n"] == 7 and target["meta"]["x"] == "y"
    assert torch.equal(target["b"], sd["b"])
    with pytest.raises(FileExistsError):
        save_state_dict(tmp_path / "ckpt", sd)
    save_state_dict(tmp_path / "ckpt", sd, save_overwrite=True)


def test_metadata_is_readable_under_reference_module_path(tmp_path):
    save_state_dict(tmp_path / "c", {"model": {"w": torch.ones(2, 2)}})
    raw = (tmp_path / "c" / ".metadata").read_bytes()
    assert b"olmo_core.distributed.checkpoint.filesystem" in raw
    md = pickle.loads(raw)  # resolves through the ``olmo_core`` alias package
    info = md.storage_data[next(iter(md.storage_data))]
    assert info.relative_path.endswith(".distcp") and info.length > 0
    assert "model.w" in get_checkpoint_metadata(tmp_path / "c").state_dict_metadata


def test_async_save(tmp_path):
    sd = {"model": {"w": torch.randn(8, 8)}}
    fut = async_save_state_dict(tmp_path / "c", sd)
    fut.result()
    (w,) = load_keys(tmp_path / "c", ["model.w"])
    assert torch.equal(w, sd["model"]["w"])


def test_model_and_optim_round_trip(tmp_path):
    model = _tiny_model(0)
    optim = AdamWConfig(lr=1e-3).build(model)
    _train_a_little(model, optim)
    save_model_and_optim_state(tmp_path / "c", model, optim, flatten_optimizer_state=True)
    keys = set(get_checkpoint_metadata(tmp_path / "c").state_dict_metadata)
    assert "model.embeddings.weight" in keys
    assert "optim.state.embeddings.weight.exp_avg" in keys and "optim.param_groups.embeddings.weight.lr" in keys

    model2 = _tiny_model(1)
    optim2 = AdamWConfig(lr=5e-4).build(model2)
    load_model_and_optim_state(tmp_path / "c", model2, optim2)
    for (n, p), (_, q) in zip(model.named_parameters(), model2.named_parameters()):
        assert torch.equal(p, q), n
        for f in ("exp_avg", "exp_avg_sq", "step"):
            assert torch.equal(torch.as_tensor(optim.state[p][f]), torch.as_tensor(optim2.state[q][f])), (n, f)
    assert optim2.param_groups[0]["lr"] == 1e-3
    # both continue identically
    _train_a_little(model, optim, seed=3)
    _train_a_little(model2, optim2, seed=3)
    for p, q in zip(model.parameters(), model2.parameters()):
        assert torch.equal(p, q)


@pytest.mark.parametrize("strategy", ["one_file", "one_file_per_tensor", "chunks"])
def test_unshard(tmp_path, strategy):
    model = _tiny_model(0)
    optim = AdamWConfig(lr=1e-3).build(model)
    _train_a_little(model, optim, steps=1)
    save_model_and_optim_state(tmp_path / "c", model, optim)
    strat = {"one_file": UnshardStrategy.one_file(), "one_file_per_tensor": UnshardStrategy.one_file_per_tensor(),
             "chunks": UnshardStrategy.chunks(1 << 20)}[strategy]
    model_path, optim_path = unshard_checkpoint(tmp_path / "c", tmp_path / "u", unshard_strategy=strat, quiet=True)
    full = dict(model.named_parameters())
    if strategy == "one_file":
        sd = torch.load(model_path, weights_only=False)
        assert set(full) <= set(sd) and all(torch.equal(sd[n], p) for n, p in full.items())
        osd = torch.load(optim_path, weights_only=False)
        assert torch.is_tensor(osd["state.embeddings.weight.exp_avg"])
    else:
        assert optim_path is None and model_path.is_dir()
        merged = {}
        for f in sorted(model_path.iterdir()):
            merged.update(torch.load(f, weights_only=False))
        assert all(torch.equal(merged[n], p) for n, p in full.items())
        if strategy == "chunks":
            assert len(list(model_path.iterdir())) > 1


def test_key_utilities():
    sd = {"model": {"a.w": torch.ones(1), "b.w": torch.zeros(1)},
          "optim": {"state.a.w.exp_avg": torch.ones(1), "param_groups.a.w.lr": 0.1, "state.b.w.exp_avg": torch.zeros(1)}}
    swap_param_keys(sd, {"a.w": "z.w"}, quiet=True)
    assert set(sd["model"]) == {"z.w", "b.w"}
    assert {"state.z.w.exp_avg", "param_groups.z.w.lr", "state.b.w.exp_avg"} == set(sd["optim"])
    swap_param_keys(sd, {"a.w": "z.w"}, reverse=True, quiet=True)
    assert set(sd["model"]) == {"a.w", "b.w"}
    pruned = prune_state_dict(sd, {"model.a.w", "optim.state.a.w.exp_avg"})
    assert "model.b.w" in pruned and set(sd["model"]) == {"a.w"} and set(sd["optim"]) == {"state.a.w.exp_avg"}
    lhs = {"x": {"a": 1}, "y": 2}
    merge_state_dicts(lhs, {"x": {"b": 3}, "y": 4})
    assert lhs == {"x": {"a": 1, "b": 3}, "y": 4}


# -- multi-rank: write with two ranks, read with one (and the other way round) ---------------------------
def _save_sharded(path):
    model = _tiny_model(0, sharded=True)
    optim = AdamWConfig(lr=1e-3).build(model)
    _train_a_little(model, optim, steps=1, seed=dist.get_rank())
    save_model_and_optim_state(path, model, optim)
    # the full parameter, for the single-process check
    rt = model._sharding_runtime
    if dist.get_rank() == 0:
        full = {s.name: rt.lowp[s.full_offset: s.full_offset + s.full_numel].view(s.full_shape).clone()
                for s in rt.slots if s.aware}
        torch.save(full, f"{path}-full.pt")


def _load_sharded(path):
    model = _tiny_model(5, sharded=True)
    optim = AdamWConfig(lr=1e-3).build(model)
    load_model_and_optim_state(path, model, optim)
    ref = torch.load(f"{path}-ref.pt", weights_only=False)
    rt = model._sharding_runtime
    for s in rt.slots:
        want = ref[s.name]
        if s.sharded:
            want = want.narrow(0, s.row_start, s.local_rows)
        assert torch.equal(s.param.data, want), s.name
        if s.aware:  # the resident compute copy was refreshed on every rank
            assert torch.equal(rt.lowp[s.full_offset: s.full_offset + s.full_numel].view(s.full_shape), ref[s.name])


def test_reshard_two_ranks_to_one(tmp_path):
    path = str(tmp_path / "c")
    run_distributed_test(_save_sharded, world_size=2, func_args=(path,))
    assert any(p.name.startswith("__1_") for p in (tmp_path / "c").iterdir())
    full = torch.load(f"{path}-full.pt", weights_only=False)
    model = _tiny_model(9)
    optim = AdamWConfig(lr=1e-3).build(model)
    load_model_and_optim_state(path, model, optim)
    for n, p in model.named_parameters():
        if n in full:
            assert torch.equal(p.data, full[n]), n
    (emb,) = load_keys(path, ["model.embeddings.weight"])
    assert torch.equal(emb, full["embeddings.weight"])


def test_reshard_one_rank_to_two(tmp_path):
    path = str(tmp_path / "c")
    model = _tiny_model(0)
    optim = AdamWConfig(lr=1e-3).build(model)
    _train_a_little(model, optim, steps=1)
    save_model_and_optim_state(path, model, optim)
    torch.save({n: p.data.clone() for n, p in model.named_parameters()}, f"{path}-ref.pt")
    run_distributed_test(_load_sharded, world_size=2, func_args=(path,))


@pytest.mark.parametrize("flatten", [False, True])
def test_optimizer_state_layouts_round_trip(tmp_path, flatten):
    """Both on-disk layouts of the optimizer state load, whatever layout the loading call asks for."""
    from olmo_core_b200.distributed.checkpoint import UNFLATTENED_MARKER, get_checkpoint_metadata

    path = str(tmp_path / "c")
    model = _tiny_model(0)
    optim = AdamWConfig(lr=3e-3, weight_decay=0.05).build(model)
    _train_a_little(model, optim, steps=2)
    save_model_and_optim_state(path, model, optim, flatten_optimizer_state=flatten)
    keys = set(get_checkpoint_metadata(path).state_dict_metadata.keys())
    assert (UNFLATTENED_MARKER in keys) == (not flatten)
    assert "optim.state.embeddings.weight.exp_avg" in keys
    model2 = _tiny_model(4)
    optim2 = AdamWConfig(lr=1.0, weight_decay=0.5).build(model2)
    load_model_and_optim_state(path, model2, optim2, flatten_optimizer_state=not flatten)
    assert optim2.param_groups[0]["lr"] == pytest.approx(3e-3) and optim2.param_groups[0]["weight_decay"] == pytest.approx(0.05)
    for (n, p), (_, q) in zip(model.named_parameters(), model2.named_parameters()):
        assert torch.equal(p.data, q.data), n
        assert torch.equal(optim.state[p]["exp_avg"], optim2.state[q]["exp_avg"]), n
