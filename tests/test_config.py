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


def test_diff_and_critical_attributes():
    a, b = Exp(), Exp()
    assert a.diff(b) == []
    b.sched.lr = 0.2
    b.model_cfg.hidden = 16
    d = {k: (x, y) for k, x, y in a.diff(b)}
    assert d["sched.lr"] == ("0.1", "0.2") and d["model_cfg.hidden"] == ("8", "16")   # printable values
    assert "optimizer_cfg.optimizer_cfg.lr" in d                 # a Ref follows its target

    class Guarded(Exp):
        _critical_attrs = ("model_cfg.hidden",)

    g = Guarded()
    g.assert_critical_attrs_expected(g.to_dict(rep=True))
    saved = g.to_dict(rep=True)
    g.sched.lr = 5.0                                             # not critical: may change between runs
    g.assert_critical_attrs_expected(saved)
    g.model_cfg.hidden = 32
    with pytest.raises(AssertionError, match="model_cfg.hidden"):
        g.assert_critical_attrs_expected(saved)


def test_mock_imports_stands_in_for_missing_packages_only(tmp_path):
    import sys

    from steptronoss_b200.config.mock_imports import get_object_from_file, mock_imports

    f = tmp_path / "needs_heavy.py"
    f.write_text(
        "import json\n"
        "import not_installed_pkg_xyz\n"
        "from not_installed_pkg_xyz.sub.mod import Thing, helper\n"
        "class Child(Thing):\n    pass\n"
        "VALUE = helper(3).whatever\n"
        "class Exp:\n    tag = json.dumps([1])\n")
    with pytest.raises(ModuleNotFoundError):
        get_object_from_file(str(f), "Exp")
    with mock_imports("not_installed_pkg_xyz", "json"):
        exp = get_object_from_file(str(f), "Exp")
        assert exp.tag == "[1]"                                   # json is installed: the real module was used
        assert list(sys.modules["not_installed_pkg_xyz"].anything) == []
    assert not any(n.startswith("not_installed_pkg_xyz") for n in sys.modules)


def test_cfshow_prints_subtrees_diffs_and_the_check_result(tmp_path):
    import io

    from steptronoss_b200.config.cfshow import show

    base = tmp_path / "base_exp_file.py"
    base.write_text(
        "from steptronoss_b200.config import Config\n"
        "class M(Config):\n    hidden: int = 8\n    layers: int\n"
        "class Base(Config):\n    model_cfg = M\n    seed = 1\n"
        "    def __init__(self):\n        super().__init__()\n        self.model_cfg.layers = 2\n"
        "class Exp(Base):\n    seed = 7\n"
        "    def __init__(self):\n        super().__init__()\n        self.model_cfg.hidden = 16\n")
    out = io.StringIO()
    assert show(str(base), out=out) == 0
    text = out.getvalue()
    assert "hidden" in text and "16" in text and "sanity_check: OK" in text
    out = io.StringIO()
    show(str(base), key="model_cfg", diff="parent", out=out)
    text = out.getvalue()
    assert text.startswith("M @") and "model_cfg.hidden: 16 | 8" in text and "seed: 7 | 1" in text
    out = io.StringIO()
    show(str(base), key="model_cfg.hidden", check=False, out=out)
    assert out.getvalue().strip() == "16"
    broken = tmp_path / "broken_exp_file.py"
    broken.write_text("from steptronoss_b200.config import Config\nclass M(Config):\n    layers: int\n"
                      "class Exp(Config):\n    model_cfg = M\n")
    out = io.StringIO()
    assert show(str(broken), out=out) == 1 and "sanity_check: FAILED" in out.getvalue() and "layers" in out.getvalue()


def test_repr_of_a_child_that_borrows_a_method_from_its_parent_terminates():
    from steptronoss_b200.config import Config, Ref

    class Child(Config):
        def __init__(self):
            super().__init__()
            self.act = Ref("..activation")
            self.owner = Ref("..")

    class Parent(Config):
        child = Child

        def activation(self, x):
            return x + 1

    p = Parent()
    text = repr(p)
    assert "<method Parent.activation>" in text and "<Parent>" in text
    assert p.child.act(1) == 2
