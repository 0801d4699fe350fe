"""Module owner protocols: where a name may live, what assignment does to it, how parameters,
buffers and children are enumerated, how device / dtype transforms keep Python identity, and how
state loads are staged and rolled back.
(reference project: tests/spec/nn/test_owner_protocols.py, test_module_registration.py,
test_state_dict_contracts.py, tests/python/test_module_buffers.py, test_module_cast.py)"""
import numpy as np
import pytest

import orthon_b200 as ob
from orthon_b200 import nn


def T(a, dtype=None):
    return ob.from_numpy(np.asarray(a, dtype=np.float32), dtype)


class Leaf(nn.Module):
    def __init__(self):
        super().__init__()
        self.weight = nn.Parameter(T([[1.0, 2.0], [3.0, 4.0]]))
        self.register_buffer("running", T([0.5, 0.5]))
        self.register_buffer("steps", ob.cast(T([3.0]), "int64"))
        self.register_buffer("scratch", T([9.0]), persistent=False)
        self.note = "plain"


class Tree(nn.Module):
    def __init__(self):
        super().__init__()
        self.left = Leaf()
        self.right = Leaf()
        self.bias = nn.Parameter(T([0.0, 0.0]))


# ---------------------------------------------------------------- registration
@pytest.mark.parametrize("kind", ["parameter", "buffer", "module"])
@pytest.mark.parametrize("name,error", [(3, TypeError), ("", ValueError), ("a.b", ValueError), ("has space", ValueError),
                                         ("forward", KeyError), ("training", KeyError), ("_parameters", KeyError)])
def test_member_names_are_validated(kind, name, error):
    m = nn.Module()
    value = {"parameter": T([1.0]), "buffer": T([1.0]), "module": nn.Module()}[kind]
    register = {"parameter": m.register_parameter, "buffer": m.register_buffer, "module": m._register_module}[kind]
    with pytest.raises(error):
        register(name, value)
    assert not m._parameters and not m._buffers and not m._modules


def test_decimal_names_are_for_children_only():
    m = nn.Module()
    m._register_module("0", nn.Module())
    assert list(m._modules) == ["0"]
    with pytest.raises(ValueError):
        m.register_parameter("0", T([1.0]))
    with pytest.raises(ValueError):
        m.register_buffer("1", T([1.0]))


@pytest.mark.parametrize("value,error", [(1.0, TypeError), ("x", TypeError), (nn.Module(), TypeError)])
def test_buffers_hold_tensors_or_none(value, error):
    m = nn.Module()
    with pytest.raises(error):
        m.register_buffer("b", value)
    m.register_buffer("b", None)
    assert "b" in m._buffers and list(m.named_buffers()) == [] and m.b is None


def test_register_parameter_requires_a_tensor_and_child_a_module():
    m = nn.Module()
    with pytest.raises(TypeError):
        m.register_parameter("w", 3.0)
    with pytest.raises(TypeError):
        m._register_module("c", T([1.0]))
    with pytest.raises(TypeError):
        nn.Parameter([1.0, 2.0])


def test_buffer_registration_refuses_names_already_in_use():
    m = Leaf()
    for taken in ("weight", "note"):
        with pytest.raises(KeyError):
            m.register_buffer(taken, T([1.0]))
    t = Tree()
    with pytest.raises(KeyError):
        t.register_buffer("left", T([1.0]))
    m.register_buffer("running", T([7.0, 7.0]))          # re-registering a buffer is allowed
    assert m.running.tolist() == [7.0, 7.0]


@pytest.mark.parametrize("value", ["text", 5, nn.Parameter(ob.from_numpy(np.ones(1, dtype=np.float32))), nn.Module()])
def test_a_buffer_slot_keeps_its_role(value):
    m = Leaf()
    with pytest.raises((KeyError, TypeError)):
        m.running = value
    assert "running" in m._buffers and m.running.tolist() == [0.5, 0.5]


def test_assigning_a_tensor_to_a_buffer_slot_replaces_the_buffer_and_keeps_persistence():
    m = Leaf()
    m.scratch = T([1.0, 2.0])
    m.running = T([4.0, 4.0])
    assert "scratch" in m._non_persistent_buffers and "running" not in m._non_persistent_buffers
    assert "scratch" not in m.state_dict() and m.state_dict()["running"].tolist() == [4.0, 4.0]
    m.running = None
    assert m.running is None and "running" not in m.state_dict() and "running" in m._buffers


@pytest.mark.parametrize("first,second", [("parameter", "module"), ("module", "parameter"), ("parameter", "attribute"),
                                           ("module", "attribute"), ("attribute", "parameter"), ("attribute", "module")])
def test_reassignment_moves_a_name_between_registries(first, second):
    make = {"parameter": lambda: nn.Parameter(T([1.0])), "module": lambda: nn.Module(), "attribute": lambda: "plain"}
    table = {"parameter": "_parameters", "module": "_modules"}
    m = nn.Module()
    m.slot = make[first]()
    m.slot = make[second]()
    for kind, registry in table.items():
        assert ("slot" in getattr(m, registry)) == (kind == second)
    assert ("slot" in m.__dict__) == (second == "attribute")


def test_plain_tensors_are_attributes_not_parameters():
    m = nn.Module()
    m.cache = T([1.0])
    assert "cache" in m.__dict__ and not list(m.parameters()) and not m.state_dict()


def test_parameter_marks_the_tensor_trainable_and_registers_the_tensor_itself():
    t = T([1.0, 2.0])
    m = nn.Module()
    m.w = nn.Parameter(t)
    assert m.w is t and t.requires_grad and t.is_leaf


def test_missing_attribute_names_the_class():
    with pytest.raises(AttributeError, match="Leaf"):
        Leaf().nothing


def test_descriptors_can_veto_before_anything_moves():
    class Guarded(nn.Module):
        @property
        def fixed(self):
            return 1

    g = Guarded()
    with pytest.raises(AttributeError):
        g.fixed = 2
    with pytest.raises(KeyError):
        g.fixed = nn.Parameter(T([1.0]))
    assert not g._parameters


# ----------------------------------------------------------------- enumeration
def test_enumeration_order_and_paths():
    t = Tree()
    assert [k for k, _ in t.named_parameters()] == ["bias", "left.weight", "right.weight"] or \
        [k for k, _ in t.named_parameters()] == ["left.weight", "right.weight", "bias"]
    keys = list(t.state_dict())
    assert set(keys) == {"bias", "left.weight", "left.running", "left.steps", "right.weight", "right.running", "right.steps"}
    assert [k for k, _ in t.named_buffers()].count("left.scratch") == 1     # non-persistent buffers are buffers, not state
    assert [k for k, _ in t.named_parameters(prefix="model")][0].startswith("model.")
    assert len(list(t.modules())) == 3 and len(list(t.children())) == 2
    assert [k for k, _ in t.named_buffers(recurse=False)] == []


def test_tied_parameters_are_one_owner_with_every_path():
    t = Tree()
    t.right.weight = nn.Parameter(t.left.weight)
    assert len(list(t.parameters())) == 2
    assert {k for k, _ in t.named_parameters()} == {"bias", "left.weight", "right.weight"}
    assert t.state_dict()["left.weight"] is t.state_dict()["right.weight"]


def test_shared_children_and_cycles_are_walked_once():
    t = Tree()
    t.again = t.left
    assert len(list(t.modules())) == 3
    assert len(list(t.parameters())) == 3
    loop = nn.Module()
    loop.me = loop
    assert list(loop.modules()) == [loop]
    assert "left.weight" in t.state_dict() and "again.weight" in t.state_dict()


def test_state_dict_returns_live_references():
    m = Leaf()
    state = m.state_dict()
    assert state["weight"] is m.weight and state["running"] is m.running
    m.weight.fill_(0.0)
    assert state["weight"].tolist() == [0.0] * 4


# ------------------------------------------------------------------- modes
def test_train_eval_reach_every_module_once():
    t = Tree()
    assert t.eval() is t and not t.training and not t.left.training and not t.right.training
    assert t.train() is t and t.left.training
    t.left.eval()
    assert t.training and not t.left.training and t.right.training


def test_zero_grad_clears_every_unique_parameter():
    t = Tree()
    (t.left.weight.sum() + t.right.weight.sum() + t.bias.sum()).backward()
    assert all(p.grad is not None for p in t.parameters())
    t.zero_grad()
    assert all(p.grad is None for p in t.parameters())


# -------------------------------------------------------------- transforms
@pytest.mark.parametrize("method,dtype", [("half", "float16"), ("bfloat16", "bfloat16"), ("float", "float32")])
def test_dtype_transforms_keep_python_identity_and_integer_buffers(method, dtype):
    t = Tree()
    t.right.weight = nn.Parameter(t.left.weight)         # a tie must stay a tie
    owners = [id(p) for p in t.parameters()]
    (t.left.weight.sum()).backward()
    assert getattr(t, method)() is t
    assert [id(p) for p in t.parameters()] == owners
    assert t.left.weight is t.right.weight
    assert all(p.dtype == dtype and p.requires_grad and p.is_leaf for p in t.parameters())
    assert t.left.running.dtype == dtype and t.left.scratch.dtype == dtype
    assert t.left.steps.dtype == "int64"                 # integer buffers keep their dtype
    if dtype != "float32":
        assert t.left.weight.grad is None                # a new representation drops the old gradient


def test_cast_then_cast_back_preserves_values_that_fit():
    m = Leaf()
    m.half()
    m.float()
    assert m.weight.tolist() == [1.0, 2.0, 3.0, 4.0] and m.weight.dtype == "float32"


def test_to_same_device_copies_storage_but_keeps_owners():
    m = Leaf()
    w, before = m.weight, m.weight._buffer_id
    running = m.running
    m.to("cpu")
    assert m.weight is w and m.weight._buffer_id != before
    assert m.running is not running and m.running.tolist() == running.tolist()


def test_buffer_tied_to_a_parameter_stays_tied_through_transforms():
    m = nn.Module()
    m.w = nn.Parameter(T([1.0, 2.0]))
    m.register_buffer("view", m.w)
    m.half()
    assert m.view is m.w and m.view.dtype == "float16"


def test_transform_failure_mutates_nothing():
    m = Leaf()
    before = (m.weight._buffer_id, m.running._buffer_id)
    with pytest.raises(Exception):
        m.cast("no-such-dtype")
    assert (m.weight._buffer_id, m.running._buffer_id) == before and m.weight.dtype == "float32"


# --------------------------------------------------------------- state loads
def test_load_state_dict_copies_values_and_replaces_buffers():
    a, b = Leaf(), Leaf()
    with ob.no_grad():
        b.weight.fill_(7.0)
        b.running.fill_(1.5)
    w, running = a.weight, a.running
    assert a.load_state_dict(b.state_dict()) is a
    assert a.weight is w and a.weight.tolist() == [7.0] * 4
    assert a.running is not running and a.running.tolist() == [1.5, 1.5]      # buffers are re-registered with copies
    b.weight.fill_(0.0)
    assert a.weight.tolist() == [7.0] * 4                                      # no aliasing with the source


@pytest.mark.parametrize("mutate,error,text", [
    (lambda s: s.pop("weight"), KeyError, "Missing keys"),
    (lambda s: s.update(extra=s["weight"]), KeyError, "Unexpected keys"),
    (lambda s: s.update(weight=ob.from_numpy(np.zeros((3, 2), dtype=np.float32))), ValueError, "size mismatch"),
    (lambda s: s.update(weight=[1.0, 2.0, 3.0, 4.0]), TypeError, "must be a Tensor"),
    (lambda s: s.update(running=None), TypeError, "must be a Tensor"),
])
def test_invalid_state_is_rejected_before_any_mutation(mutate, error, text):
    m, src = Leaf(), Leaf()
    with ob.no_grad():
        src.weight.fill_(5.0)
        src.running.fill_(5.0)
    state = dict(src.state_dict())
    mutate(state)
    with pytest.raises(error, match=text):
        m.load_state_dict(state)
    assert m.weight.tolist() == [1.0, 2.0, 3.0, 4.0] and m.running.tolist() == [0.5, 0.5]


def test_non_strict_load_takes_what_matches():
    m, src = Leaf(), Leaf()
    with ob.no_grad():
        src.running.fill_(2.0)
    m.load_state_dict({"running": src.running, "unknown": src.weight}, strict=False)
    assert m.running.tolist() == [2.0, 2.0] and m.weight.tolist() == [1.0, 2.0, 3.0, 4.0]


def test_load_casts_to_the_owner_dtype():
    m = Leaf().half()
    m.load_state_dict({k: v for k, v in Leaf().state_dict().items()})
    assert m.weight.dtype == "float16" and m.weight.tolist() == [1.0, 2.0, 3.0, 4.0]
    assert m.steps.dtype == "int64"


def test_conflicting_values_for_a_tied_parameter_are_rejected():
    t = Tree()
    t.right.weight = nn.Parameter(t.left.weight)
    state = {k: v for k, v in Tree().state_dict().items()}
    state["right.weight"] = T([[9.0, 9.0], [9.0, 9.0]])
    with pytest.raises(ValueError, match="conflicting tied parameter"):
        t.load_state_dict(state)
    state["right.weight"] = state["left.weight"]
    t.load_state_dict(state)


def test_prepared_load_rolls_back_committed_entries():
    m, src = Leaf(), Leaf()
    with ob.no_grad():
        src.weight.fill_(8.0)
        src.running.fill_(8.0)
    prepared = m._prepare_load_state_dict(src.state_dict())
    assert m.weight.tolist() == [1.0, 2.0, 3.0, 4.0]          # preparing changes nothing
    running = m.running
    prepared.commit()
    assert m.weight.tolist() == [8.0] * 4 and m.running.tolist() == [8.0, 8.0]
    prepared.rollback()
    assert m.weight.tolist() == [1.0, 2.0, 3.0, 4.0] and m.running is running


def test_load_never_consumes_gradients_or_history():
    m = Leaf()
    m.weight.sum().backward()
    g = m.weight.grad
    m.load_state_dict(Leaf().state_dict())
    assert m.weight.grad._impl_id == g._impl_id and m.weight.requires_grad and m.weight.is_leaf


# ----------------------------------------------------------------- containers
def test_sequential_registers_children_by_position():
    seq = nn.Sequential(nn.Linear(2, 3), nn.ReLU(), nn.Linear(3, 1))
    assert list(seq._modules) == ["0", "1", "2"]
    assert [k for k, _ in seq.named_parameters()] == ["0.weight", "0.bias", "2.weight", "2.bias"]
    assert seq(T([[1.0, 2.0]])).shape == (1, 1)


def test_forward_must_be_implemented():
    with pytest.raises(NotImplementedError, match="Module"):
        nn.Module()(1)


def test_repr_lists_members():
    text = repr(Tree())
    assert text.startswith("Tree(") and "(left): Leaf(" in text and "(bias): Parameter(shape=(2,))" in text
    assert repr(nn.Module()) == "Module()"
