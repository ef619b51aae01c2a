"""Smaller public names shared with the reference: data helpers, op spellings, Muon step scaling, launch monitor."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch


def test_data_helpers():
    from olmo_core_b200.data.composable.utils import path_map
    from olmo_core_b200.data.utils import (
        InstancePacker,
        SegmentTree,
        find_end_first_consecutive_true,
        find_start_last_consecutive_true,
        group_consecutive_values,
    )

    a = np.array([1, 1, 0, 1, 1, 1], dtype=bool)
    assert find_end_first_consecutive_true(a) == 2 and find_start_last_consecutive_true(a) == 3
    assert find_end_first_consecutive_true(~a) == 0 and find_start_last_consecutive_true(np.array([1, 0], dtype=bool)) == -1
    assert find_end_first_consecutive_true(np.ones(4, dtype=bool)) == 4
    assert [g.tolist() for g in group_consecutive_values(np.array([1, 2, 3, 7, 8, 10]))] == [[1, 2, 3], [7, 8], [10]]

    tree = SegmentTree(8)  # a fresh instance (8 free tokens) always fits
    assert tree.query(3).leaf_id == 7 and tree.root_node.weight == 8
    tree.leaf_nodes[4].update(5)  # some instance has 5 free tokens: the tightest fit for 3
    assert tree.query(3).leaf_id == 4 and tree.query(6).leaf_id == 7
    tree.leaf_nodes[2].update(3)
    assert tree.query(3).leaf_id == 2
    tree.leaf_nodes[2].update(0)
    assert tree.query(3).leaf_id == 4 and tree.query(3).is_leaf and not tree.root_node.is_leaf
    with pytest.raises(AssertionError):
        SegmentTree(6)

    packer = InstancePacker(8)
    for i, n in enumerate([5, 3, 4]):
        packer.pack_document(i, n)
    assert packer.instance_bins == [[0, 1], [2]] and packer.total_tokens == 12 and packer.total_padding == 4
    packer.reset()
    assert packer.instance_bins == []
    assert path_map(len, ["a", "bb", "ccc"], max_workers=2) == [1, 2, 3] and path_map(len, ["a"], max_workers=0) == [1]


def test_long_document_iteration(tmp_path):
    from olmo_core_b200.data.utils import iter_document_indices, iter_document_indices_with_max_sequence_length

    eos = 0
    data = np.array([5, 6, 7, 8, 9, 10, 11, eos, 3, 4, eos], dtype=np.uint16)
    path = tmp_path / "d.npy"
    data.tofile(path)
    plain = list(iter_document_indices(path, eos_token_id=eos, dtype=np.uint16))
    assert plain == [(0, 8), (8, 11)]
    cut = list(iter_document_indices_with_max_sequence_length(path, 3, eos_token_id=eos, dtype=np.uint16))
    assert cut == [(0, 3), (8, 11)]
    parts = list(iter_document_indices_with_max_sequence_length(path, 3, eos_token_id=eos, dtype=np.uint16,
                                                                long_doc_strategy="fragment"))
    assert parts == [(0, 3), (3, 6), (6, 8), (8, 11)]


def test_moe_op_spellings_and_aux_loss():
    from olmo_core_b200.kernels.moe import assert_equal, assert_is_matrix, assert_is_vector
    from olmo_core_b200.ops import AutoAuxiliaryLoss, attach_auxiliary_loss
    from olmo_core_b200.ops import moe as ops

    x = torch.randn(6, 4)
    top = torch.tensor([[0, 1], [1, 2], [2, 0], [0, 2], [1, 0], [2, 1]])
    indices, bin_ids, bins = ops.indices_and_bins(top, 3)
    got = ops.GatherOp.apply(x, indices, bin_ids, bins, 2)
    torch.testing.assert_close(got, ops.gather(x, indices, bin_ids, bins, 2))
    back = ops.ScatterOp.apply(got, indices, bin_ids, None, bins, 2)
    torch.testing.assert_close(back, 2 * x)  # each token comes back once per copy
    binned = ops.BinnedGatherOp.apply(x, indices, bins, 4, 2)
    assert binned.shape == (3, 4, 4)
    torch.testing.assert_close(ops.BinnedScatterOp.apply(binned, indices, None, bins, 2), 2 * x)
    assert ops.AllToAllOp is not None

    assert_is_matrix(x)
    assert_is_vector(x[0])
    assert_equal(3, 3)
    with pytest.raises(ValueError):
        assert_is_vector(x)
    with pytest.raises(ValueError):
        assert_equal(3, 4)

    act = torch.ones(3, requires_grad=True)
    aux = torch.tensor(2.0, requires_grad=True) * 3
    aux.retain_grad()
    out = attach_auxiliary_loss(act * 1.0, aux)
    out.sum().backward()
    assert float(aux.grad) == 1.0 and AutoAuxiliaryLoss.apply is not None


def test_muon_step_scaling_and_cautious_decay():
    from olmo_core_b200.optim.muon import Muon, MuonAdjustLRStrategy, MuonConfig, newton_schulz

    assert MuonAdjustLRStrategy.spectral_norm.scale(8, 2) == 2.0 and MuonAdjustLRStrategy.spectral_norm.scale(2, 8) == 1.0
    assert MuonAdjustLRStrategy.rms_norm.scale(4, 16) == pytest.approx(0.8)
    cfg = MuonConfig()
    assert (cfg.lr, cfg.weight_decay, cfg.nesterov, cfg.adjust_lr) == (0.01, 0.1, False, MuonAdjustLRStrategy.rms_norm)

    torch.manual_seed(0)
    w0, g = torch.randn(4, 16), torch.randn(4, 16)
    ortho = newton_schulz(g.clone(), 5)

    def one_step(**kw):
        p = torch.nn.Parameter(w0.clone())
        opt = Muon([p], lr=0.1, mu=0.0, nesterov=False, weight_decay=0.0, **kw)
        p.grad = g.clone()
        opt.step()
        return p.detach()

    torch.testing.assert_close(one_step(adjust_lr="rms_norm"), w0 - 0.1 * 0.8 * ortho)
    torch.testing.assert_close(one_step(adjust_lr="spectral_norm"), w0 - 0.1 * ortho)
    torch.testing.assert_close(one_step(adjust_lr=None), w0 - 0.1 * ortho)

    p = torch.nn.Parameter(w0.clone())
    opt = Muon([p], lr=0.1, mu=0.0, nesterov=False, weight_decay=0.5, adjust_lr=None, cautious_wd=True)
    p.grad = g.clone()
    opt.step()
    decayed = torch.where(ortho * w0 > 0, w0 * (1 - 0.05), w0)
    torch.testing.assert_close(p.detach(), decayed - 0.1 * ortho)


def test_launch_monitor_timeouts_and_host_occupancy():
    from olmo_core_b200.launch.beaker import GantryMonitorCallback
    from olmo_core_b200.launch.select_beaker_hosts import node_is_occupied

    now = [0.0]
    sent, stops = [], []
    cb = GantryMonitorCallback(None, step_timeout=600, step_soft_timeout=120, warning_frequency=300, workload_name="me/run",
                               send=sent.append, interrupt=lambda: stops.append(now[0]), clock=lambda: now[0])
    cb.on_start()
    assert "has started" in sent[-1]
    now[0] = 1000.0  # no step seen yet, but the run is younger than the start-up grace periods: nothing happens
    cb.on_no_new_logs()
    assert len(sent) == 1 and not stops
    cb.on_log(log_line="[step=10/100,epoch=1] train/loss=2.5")
    now[0] = 1100.0
    cb.on_log(log_line="some other line")
    assert len(sent) == 1
    now[0] = 1130.0  # 130 s without a step: one warning ...
    cb.on_no_new_logs()
    assert "hasn't stepped recently" in sent[-1] and len(sent) == 2
    now[0] = 1200.0  # ... and no second one inside the warning interval
    cb.on_no_new_logs()
    assert len(sent) == 2 and not stops
    now[0] = 1700.0  # 700 s without a step: the workload is stopped
    cb.on_no_new_logs()
    assert stops == [1700.0] and "failed to step in time" in sent[-1]

    job = lambda slots, priority, preemptible: SimpleNamespace(  # noqa: E731
        assignment_details=SimpleNamespace(resource_assignment=SimpleNamespace(assigned_slots_count=slots)),
        priority=priority, preemptible=preemptible)
    beaker = lambda jobs: SimpleNamespace(job=SimpleNamespace(list=lambda scheduled_on_node: jobs))  # noqa: E731
    assert node_is_occupied(beaker([]), "n", "normal") == ("n", False)
    assert node_is_occupied(beaker([job(8, "low", True)]), "n", "normal") == ("n", False)   # we may preempt it
    assert node_is_occupied(beaker([job(8, "high", True)]), "n", "normal") == ("n", True)
    assert node_is_occupied(beaker([job(8, "low", False)]), "n", "normal") == ("n", True)
    assert node_is_occupied(beaker([job(0, "high", False)]), "n", "normal") == ("n", False)  # holds no slots
