"""Foundation layer: config system (typed decoding, overrides, registries), io on local paths, assorted utils, eval metrics."""

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import pytest
import torch

from olmo_core_b200 import io
from olmo_core_b200.config import Config, DType, Registrable, StrEnum
from olmo_core_b200.exceptions import OLMoConfigurationError


class Color(StrEnum):
    red = "red"
    blue = "blue"


@dataclass
class Inner(Config):
    width: int = 4
    color: Color = Color.red
    dims: Tuple[int, ...] = (1, 2)


@dataclass
class Outer(Config):
    inner: Inner = field(default_factory=Inner)
    items: List[Inner] = field(default_factory=list)
    table: Dict[str, float] = field(default_factory=dict)
    name: Optional[str] = None
    dtype: DType = DType.bfloat16


def test_config_round_trip_and_typed_decoding():
    cfg = Outer(inner=Inner(width=8, color=Color.blue), items=[Inner(), Inner(width=2)], table={"a": 1.5}, name="x")
    data = cfg.as_config_dict()
    assert data["inner"]["color"] == "blue" and data["_CLASS_"].endswith("Outer")
    back = Outer.from_dict(data)
    assert back == cfg and isinstance(back.inner.color, Color) and isinstance(back.inner.dims, tuple)
    assert back.dtype.as_pt() == torch.bfloat16 and DType.from_pt(torch.float32) == DType.float32
    assert str(Color.red) == "red"


def test_config_overrides():
    cfg = Outer(items=[Inner(), Inner()])
    new = cfg.merge(["inner.width=16", "--inner.color=blue", "items.1.width=3", "name=null", "table.b=2.5"])
    assert new.inner.width == 16 and new.inner.color == Color.blue and new.items[1].width == 3
    assert new.name is None and new.table["b"] == 2.5
    assert cfg.inner.width == 4  # merge returns a new object
    with pytest.raises(Exception):
        cfg.merge(["inner.no_such_field=1"])
    assert cfg.replace(name="y").name == "y"
    seen = []
    cfg.apply(lambda c: seen.append(type(c).__name__))
    assert seen.count("Inner") == 3 and "Outer" in seen


def test_registrable_dispatches_on_name():
    class Shape(Config, Registrable):
        pass

    @Shape.register("square")
    @dataclass
    class Square(Shape):
        side: float = 1.0

    @Shape.register("circle")
    @dataclass
    class Circle(Shape):
        radius: float = 1.0

    assert Shape.get_registered_class("circle") is Circle and Circle.get_registered_name() == "circle"
    assert set(Shape.get_registered_names()) >= {"square", "circle"}
    with pytest.raises(Exception):
        Shape.get_registered_class("triangle")


def test_local_io(tmp_path):
    assert io.is_url("s3://bucket/key") and io.is_url("https://x/y") and not io.is_url("/tmp/x") and not io.is_url("rel/x")
    assert io.join_path("s3://b/a/", "c") == "s3://b/a/c" and str(io.join_path(tmp_path, "c")) == str(tmp_path / "c")
    p = tmp_path / "dir" / "f.bin"
    io.write_bytes(p, b"0123456789")
    assert io.file_exists(p) and io.get_file_size(p) == 10 and io.get_bytes_range(p, 2, 3) == b"234"
    with pytest.raises(FileExistsError):
        io.write_bytes(p, b"x", overwrite=False)
    io.write_text(tmp_path / "dir" / "t.txt", "hello")
    assert io.read_text(tmp_path / "dir" / "t.txt") == "hello"
    assert sorted(map(str, io.list_directory(tmp_path / "dir"))) == sorted([str(p), str(tmp_path / "dir" / "t.txt")])
    assert [s for s in io.glob_directory(str(tmp_path / "dir" / "*.bin"))] == [str(p)]
    io.copy_file(p, tmp_path / "copy.bin")
    assert io.read_bytes(tmp_path / "copy.bin") == b"0123456789"
    io.copy_dir(tmp_path / "dir", tmp_path / "dir2")
    assert not io.dir_is_empty(tmp_path / "dir2")
    io.clear_directory(tmp_path / "dir2")
    assert io.dir_is_empty(tmp_path / "dir2") and io.dir_is_empty(tmp_path / "missing")
    io.remove_file(p)
    assert not io.file_exists(p)
    obj = {"a": [1, 2, 3]}
    assert io.deserialize_from_tensor(io.serialize_to_tensor(obj)) == obj


def test_utils():
    from datetime import timedelta

    from olmo_core_b200 import utils

    assert utils.flatten_dict({"a": {"b": 1, "c": {"d": 2}}, "e": 3}) == {"a.b": 1, "a.c.d": 2, "e": 3}
    assert list(utils.roundrobin("ABC", "D", "EF")) == list("ADEBFC")
    assert utils.powers_of_2(20) == [16, 4] or sum(utils.powers_of_2(20)) == 20
    assert utils.ensure_multiple_of(100, 64) == 128 and utils.ensure_multiple_of(128, 64) == 128
    assert utils.format_int(1_500_000).upper().endswith("M") and utils.get_element_size(torch.bfloat16) == 2
    assert "1" in utils.format_timedelta(timedelta(hours=1, minutes=2))
    moved = utils.move_to_device({"x": torch.ones(2), "y": [torch.zeros(1)], "z": 3}, torch.device("cpu"))
    assert moved["z"] == 3 and moved["y"][0].device.type == "cpu"
    assert list(utils.threaded_generator(iter(range(5)))) == [0, 1, 2, 3, 4]
    assert utils.same_storage(torch.ones(4)[:2], torch.ones(4)) is False


def test_lm_evaluator_reports_loss_and_perplexity_per_label():
    from olmo_core_b200.eval import LMEvaluator

    batches = [
        {"input_ids": torch.zeros(2, 4, dtype=torch.long), "metadata": [{"label": "a"}, {"label": "b"}]},
        {"input_ids": torch.zeros(2, 4, dtype=torch.long), "metadata": [{"label": "a"}, {"label": "a"}]},
    ]
    ev = LMEvaluator(name="val", batches=batches, labels=["a", "b"], device=torch.device("cpu"))
    ce = [torch.tensor([[1.0, 1.0, 1.0], [3.0, 3.0, 3.0]]), torch.tensor([[2.0, 2.0, 2.0], [2.0, 2.0, 2.0]])]
    for batch, loss in zip(ev, ce):
        ev.update_metrics(batch, loss, None)
    metrics = {k: float(v) for k, v in ev.compute_metrics().items()}
    assert metrics["a/CE loss"] == pytest.approx((1.0 + 2.0 + 2.0) / 3)
    assert metrics["b/CE loss"] == pytest.approx(3.0)
    assert metrics["b/PPL"] == pytest.approx(float(torch.tensor(3.0).exp()))
