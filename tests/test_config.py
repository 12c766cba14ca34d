"""Config system: typed decode of nested structures, dot-path overrides, registrable polymorphism, YAML files."""

import typing
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import pytest
import torch
import yaml

from olmax_b200.config import config_to_yaml, parse_config_from_args
from olmax_b200.types import Duration, DurationUnit, PathOrStr
from olmax_b200.utils.dataclass_codec import DecodeError, Registrable, decode, encode


@dataclass
class Foo:
    x: int


@dataclass
class Config:
    foo: Foo
    bar: Optional[Foo]
    lr: float
    path: PathOrStr
    list_data: List[Foo]
    tuple_data: Tuple[int, int]
    sequence_or_int: typing.Union[int, Sequence[int], None]
    dtype: torch.dtype = torch.float32


def _cfg():
    return Config(foo=Foo(0), bar=None, lr=0.0, path="/path", list_data=[Foo(2)], tuple_data=(0, 1), sequence_or_int=2)


def test_overrides_on_complex_types():
    cfg = parse_config_from_args(_cfg(), args=["foo.x=1", "list_data.0.x=1", "sequence_or_int=[0, 1]", "--lr=1e-3",
                                               "--dtype=bfloat16", "--bar={x: 7}"])
    assert cfg.foo.x == 1 and cfg.list_data[0].x == 1
    assert cfg.sequence_or_int == (0, 1)
    assert cfg.lr == pytest.approx(1e-3)
    assert cfg.dtype == torch.bfloat16
    assert cfg.bar == Foo(7)
    assert cfg.tuple_data == (0, 1)


def test_int_stays_int_in_union_and_bad_types_fail():
    cfg = parse_config_from_args(_cfg(), args=[])
    assert cfg.sequence_or_int == 2 and isinstance(cfg.sequence_or_int, int)
    with pytest.raises(DecodeError):
        parse_config_from_args(_cfg(), args=["foo.x=notanint"])
    with pytest.raises(DecodeError):
        parse_config_from_args(_cfg(), args=["nonexistent=3"])


def test_flag_and_dash_handling():
    @dataclass
    class C:
        use_thing: bool = False
        n: int = 1

    c = parse_config_from_args(C(), args=["--use-thing", "--n=3"])
    assert c.use_thing is True and c.n == 3


@dataclass
class Fruit(Registrable):
    calories: int = 0
    price: float = 0.0


@Fruit.register("banana")
@dataclass
class Banana(Fruit):
    calories: int = 200
    price: float = 1.25


@Fruit.register("apple")
@dataclass
class Apple(Fruit):
    calories: int = 150
    price: float = 1.50


@dataclass
class FruitBasket:
    fruit: Fruit
    count: int


def test_registrable_overrides(tmp_path):
    basket = FruitBasket(fruit=Banana(), count=2)
    path = tmp_path / "config.yaml"
    path.write_text(yaml.safe_dump(encode(basket)))
    for b in (parse_config_from_args(basket, args=["--fruit.type=apple"]),
              parse_config_from_args(path, FruitBasket, args=["--fruit.type=apple"])):
        assert isinstance(b.fruit, Apple) and b.fruit.price == basket.fruit.price
    for b in (parse_config_from_args(basket, args=["--fruit={type: apple}"]),
              parse_config_from_args(path, FruitBasket, args=["--fruit={type: apple}"])):
        assert isinstance(b.fruit, Apple) and b.fruit.price == Apple().price
    with pytest.raises(KeyError):
        parse_config_from_args(basket, args=["--fruit.type=durian"])
    with pytest.raises(ValueError):
        Fruit.register("apple")(Banana)


def test_encode_decode_roundtrip_of_real_config():
    from olmax_b200.launch.train_transformer import IntegrationTestConfig, _parse_args, build_config

    opts, overrides = _parse_args(["--recipe=olmo2_32B_bench", "--mesh-type=HSDP", "--shard-degree=1",
                                   "--global-device-count=1", "--num_microbatches=2",
                                   "--model.layer_ac_policy={type: save_only_these_names, names: ['layers.*.mlp']}",
                                   "--env.nccl.debug=INFO"])
    cfg = build_config(opts, overrides)
    assert cfg.num_microbatches == 2 and cfg.env.nccl.debug == "INFO"
    assert cfg.model.layer_ac_policy.names == ["layers.*.mlp"]
    assert cfg.mesh.axis_names == ("fsdp_replicate", "fsdp_shard")
    again = decode(IntegrationTestConfig, yaml.safe_load(config_to_yaml(cfg)))
    assert encode(again) == encode(cfg)


def test_duration():
    assert Duration.steps(10).due(step=10, tokens=None)
    assert not Duration.steps(10).due(step=9, tokens=None)
    assert Duration.tokens(100).due(tokens=100)
    assert not Duration.epochs(1).due(epoch=1, tokens=None)
    assert Duration.epochs(1).due(epoch=2, tokens=None)
    assert decode(Duration, {"value": 3, "unit": "steps"}).unit == DurationUnit.steps
