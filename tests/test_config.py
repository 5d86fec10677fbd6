import copy
import pickle

import pytest
import torch

from steptronoss_b200.config import Config, DataClass, Ref, parse_args, recur_to_allowed_types, writable_property


class Opt(Config):
    lr: float = Ref("...sched.lr")
    name = "adam"


class GM(Config):
    optimizer_cfg: Opt = Opt
    params_dtype = Ref("..model_cfg.params_dtype")
    clip: float = 1.0


class Model(Config):
    params_dtype = torch.bfloat16
    hidden: int

    @writable_property
    def ffn(self):
        return self.hidden * 4

    def build(self):
        return "built"


class Sched(Config):
    lr: float


class Exp(Config):
    model_cfg = Model
    optimizer_cfg = GM
    sched = Sched
    seed = 1

    def __init__(self):
        super().__init__()
        self.model_cfg.hidden = 8
        self.sched.lr = 0.1
        self.extra = {"a": 1}


def test_children_are_per_instance_and_linked():
    a, b = Exp(), Exp()
    assert a.model_cfg is not b.model_cfg
    assert a.model_cfg.father() is a and a.optimizer_cfg.optimizer_cfg.root() is a
    assert a.optimizer_cfg.optimizer_cfg._get_node_name() == "Exp.optimizer_cfg.optimizer_cfg"


def test_ref_resolution_levels_and_default():
    e = Exp()
    assert e.optimizer_cfg.optimizer_cfg.lr == 0.1
    assert e.optimizer_cfg.params_dtype is torch.bfloat16
    e.sched.lr = 0.5
    assert e.optimizer_cfg.optimizer_cfg.lr == 0.5

    class X(Config):
        v = Ref("..nothing.here", 7)

    assert X().v == 7
    with pytest.raises(AttributeError):
        class Y(Config):
            v = Ref("..nothing")
        Y().v


def test_writable_property_and_methods_not_fields():
    e = Exp()
    assert e.model_cfg.ffn == 32
    e.model_cfg.ffn = 3
    assert e.model_cfg.ffn == 3
    assert "build" not in e.model_cfg.keys() and "ffn" in e.model_cfg.to_dict()


def test_merge_modify_and_strict_attrs():
    e = Exp()
    diff = e.merge({"model_cfg.hidden": 16, "seed": 1, "extra.a": 2}, exists_only=True)
    assert ("model_cfg.hidden", 8, 16) in diff and ("extra.a", 1, 2) in diff and len(diff) == 2
    with pytest.raises(KeyError):
        e.merge({"model_cfg.nope": 1}, exists_only=True)
    with e.modify(seed=5):
        assert e.seed == 5
    assert e.seed == 1
    with pytest.raises(AttributeError):
        e.bogus = 1


def test_sanity_check_required_fields():
    class M(Config):
        need: int

    class E(Config):
        m = M

    with pytest.raises(AssertionError):
        E().sanity_check()
    e = E()
    e.m.need = 1
    e.sanity_check()


def test_copy_pickle_to_dict():
    e = Exp()
    e2 = copy.deepcopy(e)
    e2.sched.lr = 0.9
    assert e.optimizer_cfg.optimizer_cfg.lr == 0.1 and e2.optimizer_cfg.optimizer_cfg.lr == 0.9
    e3 = pickle.loads(pickle.dumps(e))
    assert e3.optimizer_cfg.optimizer_cfg.lr == 0.1
    d = e.to_dict()
    assert d["model_cfg"]["hidden"] == 8 and d["optimizer_cfg"]["optimizer_cfg"]["lr"] == 0.1
    assert dict(**e.sched) == {"lr": 0.1}


def test_subclass_overrides_child_type():
    class Model2(Model):
        extra_field = 3

    class Exp2(Exp):
        model_cfg = Model2

    e = Exp2()
    assert isinstance(e.model_cfg, Model2) and e.model_cfg.hidden == 8


class S(DataClass):
    a: int = 1
    b: list = []


def test_dataclass_and_plain_types():
    s = S(a=2)
    s.b.append(1)
    assert S().b == [] and dict(**s) == {"a": 2, "b": [1]} and s["a"] == 2
    assert pickle.loads(pickle.dumps(s)) == s
    assert recur_to_allowed_types({"x": s, "e": Exp().sched}) == {"x": {"a": 2, "b": [1]}, "e": {"lr": 0.1}}


def test_parse_args():
    out = parse_args(["a.b=1", "x=foo", "--flag", "y=[1,2]", "z=1e-3", "t=True"])
    assert out == {"a.b": 1, "x": "foo", "y": [1, 2], "z": 1e-3, "t": True}
