"""Module base class: explicit registries for parameters, buffers and children.

Behavioural contract (reference project: python/orthon/nn/module.py:22-460):
* ``Parameter(t)`` marks a tensor trainable; assigning it registers the *tensor* itself, so
  ``module.weight`` is the Tensor and its Python identity survives ``to/cast/half/bfloat16``
  (the storage is rebound underneath it and any gradient is dropped).
* ``register_buffer(name, tensor, persistent=True)``; a buffer slot keeps its role until it is
  re-registered, ``None`` buffers stay registered but are skipped by enumeration.
* ``parameters()`` yields unique tensors (tied parameters once); ``named_parameters()`` yields
  every path.  ``state_dict()`` returns live references in registration order.
* ``load_state_dict`` prepares every value first and only then commits, with rollback.
"""
from .. import _C
from .._state import PreparedLoad, commit_prepared

_FLOATING = ("float16", "bfloat16", "float32", "float64")
_RESERVED = ("_parameters", "_buffers", "_modules", "_non_persistent_buffers", "training")


def _no_grad():
    import orthon_b200 as ob
    return ob.no_grad()


class Parameter:
    """Marker wrapper: ``self.w = Parameter(tensor)`` registers ``tensor`` as trainable."""

    def __init__(self, data):
        if not isinstance(data, _C.Tensor):
            raise TypeError(f"Parameter expects a Tensor, got {type(data).__name__}")
        data.requires_grad_(True)
        self._data = data


def _check_member_name(owner, name, kind):
    """Names of registered members are path components of state-dict keys: identifiers (children
    may also be decimal, for containers) that do not shadow anything the class defines."""
    if not isinstance(name, str):
        raise TypeError(f"{kind} name must be a string")
    well_formed = bool(name) and "." not in name and (name.isidentifier() or (kind == "module" and name.isdecimal()))
    if not well_formed:
        raise ValueError(f"invalid {kind} name {name!r}")
    if name in _RESERVED or hasattr(type(owner), name):
        raise KeyError(f"'{name}' is already an attribute of this module")


_EXPECTED = {"parameter": (lambda v: isinstance(v, _C.Tensor), "registered parameter must be a Tensor"),
             "module": (lambda v: isinstance(v, Module), "registered child must be a Module")}


class Module:
    """A name belongs to at most one of four places: the parameter, buffer or child registry, or
    the instance dictionary (plain attributes).  Every write goes through `_set_member`, which
    first decides whether the write is admissible and only then moves the name to its new place,
    evicting it from wherever it was."""

    def __init__(self):
        d = object.__getattribute__(self, "__dict__")
        d.update(_parameters={}, _buffers={}, _modules={}, _non_persistent_buffers=set(), training=True)

    # ------------------------------------------------------------ registration
    def _registries(self):
        return {"parameter": self._parameters, "buffer": self._buffers, "module": self._modules}

    def _admit(self, name, value, kind):
        registries = self._registries()
        if kind == "attribute":
            if name in registries["buffer"]:
                raise KeyError(f"cannot assign a {kind} to registered buffer '{name}'")
            return
        _check_member_name(self, name, kind)
        if kind == "buffer":
            plain = object.__getattribute__(self, "__dict__")
            if name in plain or name in registries["parameter"] or name in registries["module"]:
                raise KeyError(f"'{name}' is already an attribute or registered member")
            if not (value is None or isinstance(value, _C.Tensor)):
                raise TypeError(f"buffer '{name}' expects a Tensor or None, got {type(value).__name__}")
            return
        if name in registries["buffer"]:  # a buffer slot keeps its role until it is re-registered
            raise KeyError(f"cannot assign a {kind} to registered buffer '{name}'")
        accepts, complaint = _EXPECTED[kind]
        if not accepts(value):
            raise TypeError(complaint)

    def _set_member(self, name, value, kind, *, persistent=True):
        self._admit(name, value, kind)
        if kind == "attribute":
            object.__setattr__(self, name, value)  # a descriptor may still refuse: nothing has moved yet
        else:
            object.__getattribute__(self, "__dict__").pop(name, None)
        for other, table in self._registries().items():
            if other != kind:
                table.pop(name, None)
        if kind == "buffer" and not persistent:
            self._non_persistent_buffers.add(name)
        else:
            self._non_persistent_buffers.discard(name)
        if kind != "attribute":
            self._registries()[kind][name] = value

    def register_buffer(self, name, tensor, persistent=True):
        self._set_member(name, tensor, "buffer", persistent=bool(persistent))

    def register_parameter(self, name, tensor):
        self._set_member(name, tensor._data if isinstance(tensor, Parameter) else tensor, "parameter")

    def _register_module(self, name, module):
        self._set_member(name, module, "module")

    def __setattr__(self, name, value):
        if isinstance(value, Parameter):
            return self._set_member(name, value._data, "parameter")
        if isinstance(value, Module):
            return self._set_member(name, value, "module")
        if name in self._buffers:  # assignment to a buffer slot replaces the buffer, keeping its persistence
            return self._set_member(name, value, "buffer", persistent=name not in self._non_persistent_buffers)
        return self._set_member(name, value, "attribute")

    def __getattr__(self, name):
        # Called only after normal lookup failed, i.e. for registered members (and during
        # construction before __init__ ran, when the registries do not exist yet).
        own = object.__getattribute__(self, "__dict__")
        for registry in ("_parameters", "_buffers", "_modules"):
            members = own.get(registry, ())
            if name in members:
                return members[name]
        raise AttributeError(f"'{type(self).__name__}' has no attribute '{name}'")

    # --------------------------------------------------------------- traversal
    def _walk_modules(self, prefix="", *, recurse=True, unique=False):
        seen = set()

        def visit(module, path, ancestors):
            ident = id(module)
            if ident in ancestors or (unique and ident in seen):
                return
            seen.add(ident)
            yield path, module
            if recurse:
                for child_name, child in module._modules.items():
                    yield from visit(child, path + child_name + ".", ancestors | {ident})

        yield from visit(self, prefix, frozenset())

    def _state_entries(self, prefix="", *, parameters=True, buffers=True, persistent_only=True, recurse=True):
        """(key, owner module, kind, local name, tensor): parameters, then buffers, then children."""
        for path, module in self._walk_modules(prefix, recurse=recurse):
            if parameters:
                for name, tensor in module._parameters.items():
                    yield path + name, module, "parameter", name, tensor
            if buffers:
                for name, tensor in module._buffers.items():
                    if persistent_only and name in module._non_persistent_buffers:
                        continue
                    if tensor is not None:
                        yield path + name, module, "buffer", name, tensor

    def modules(self):
        for _, m in self._walk_modules(unique=True):
            yield m

    def children(self):
        return iter(self._modules.values())

    def named_parameters(self, prefix=""):
        if prefix and not prefix.endswith("."):
            prefix += "."
        for key, _, _, _, tensor in self._state_entries(prefix, buffers=False):
            yield key, tensor

    def parameters(self):
        seen = set()
        for _, tensor in self.named_parameters():
            if id(tensor) not in seen:
                seen.add(id(tensor))
                yield tensor

    def named_buffers(self, prefix="", recurse=True):
        if prefix and not prefix.endswith("."):
            prefix += "."
        for key, _, _, _, tensor in self._state_entries(prefix, parameters=False, persistent_only=False, recurse=recurse):
            yield key, tensor

    def buffers(self, recurse=True):
        seen = set()
        for _, tensor in self.named_buffers(recurse=recurse):
            if id(tensor) not in seen:
                seen.add(id(tensor))
                yield tensor

    # ------------------------------------------------------------------- modes
    def _set_training(self, flag):
        for m in self.modules():
            m.training = flag
        return self

    def train(self):
        return self._set_training(True)

    def eval(self):
        return self._set_training(False)

    def zero_grad(self):
        for p in self.parameters():
            if p.grad is not None:
                p.zero_grad()

    # --------------------------------------------------------- device / dtype
    def _apply_tensor_transform(self, transform, *, floating_buffers_only=False):
        """Transforms every unique tensor once; parameters keep their Python object, buffer
        slots are re-registered, and ties (also buffer-to-parameter ties) stay ties.  All
        conversions finish before the first mutation."""
        mods = list(self.modules())
        param_ids = {id(p) for m in mods for p in m._parameters.values()}
        owners, slots = {}, []
        for m in mods:
            for p in m._parameters.values():
                owners.setdefault(id(p), p)
            for name, b in m._buffers.items():
                if b is None:
                    continue
                if floating_buffers_only and b.dtype not in _FLOATING and id(b) not in param_ids:
                    continue
                owners.setdefault(id(b), b)
                slots.append((m, name, b))
        fresh = {}
        with _no_grad():
            for ident, tensor in owners.items():
                out = transform(tensor)
                if tuple(out.shape) != tuple(tensor.shape):
                    raise RuntimeError("model transform must preserve shape")
                if not out.is_leaf or out._impl_id == tensor._impl_id:
                    out = out.to(out.device)  # publish an independent leaf
                out.requires_grad_(tensor.requires_grad)
                fresh[ident] = out
            for ident in param_ids:
                owners[ident]._rebind_model_value_(fresh[ident])
                fresh[ident] = owners[ident]
            for m, name, original in slots:
                m._set_member(name, fresh[id(original)], "buffer", persistent=name not in m._non_persistent_buffers)
        return self

    def to(self, device):
        return self._apply_tensor_transform(lambda t: t.to(device))

    def cast(self, dtype):
        return self._apply_tensor_transform(lambda t: _C.cast(t, dtype), floating_buffers_only=True)

    def half(self):
        return self.cast("float16")

    def bfloat16(self):
        return self.cast("bfloat16")

    def float(self):
        return self.cast("float32")

    # ------------------------------------------------------------------- state
    def state_dict(self, _prefix=""):
        return {key: tensor for key, _, _, _, tensor in self._state_entries(_prefix)}

    def load_state_dict(self, state, strict=True):
        commit_prepared([self._prepare_load_state_dict(state, strict=strict)])
        return self

    def _prepare_load_state_dict(self, state, strict=True, map_location=None):
        entries = list(self._state_entries())
        have = {e[0] for e in entries}
        if strict:
            missing, unexpected = have - set(state), set(state) - have
            if missing:
                raise KeyError(f"Missing keys in state_dict: {sorted(missing)}")
            if unexpected:
                raise KeyError(f"Unexpected keys in state_dict: {sorted(unexpected)}")
        target = None if map_location is None else _C.Device(str(map_location))
        staged, first_tied = [], {}
        for key, owner, kind, local, current in entries:
            if key not in state:
                continue
            src = state[key]
            if not isinstance(src, _C.Tensor):
                raise TypeError(f"state_dict entry '{key}' must be a Tensor, got {type(src).__name__}")
            if tuple(src.shape) != tuple(current.shape):
                raise ValueError(f"size mismatch for '{key}': current {list(current.shape)} vs loaded {list(src.shape)}")
            with _no_grad():
                value = src.to(target if target is not None else current.device)  # always an independent copy
                if value.dtype != current.dtype:
                    value = _C.cast(value, current.dtype)
            if kind == "parameter":
                if id(current) in first_tied:
                    other_key, other = first_tied[id(current)]
                    a, b = other.tolist(), value.tolist()
                    if not all(x == y or (x != x and y != y) for x, y in zip(a, b)):
                        raise ValueError(f"conflicting tied parameter state: '{other_key}' and '{key}'")
                    continue
                first_tied[id(current)] = (key, value)
            staged.append((owner, kind, local, current, value))

        param_ids = {id(p) for p in self.parameters()}
        moves = []
        if target is not None:
            loaded = {(id(o), n) for o, k, n, _, _ in staged if k == "buffer"}
            moved_cache = {}
            for m in self.modules():
                for name, tensor in m._buffers.items():
                    if tensor is None or tensor.device == target or (id(m), name) in loaded:
                        continue
                    if id(tensor) in param_ids:
                        replacement = tensor
                    else:
                        if id(tensor) not in moved_cache:
                            with _no_grad():
                                nv = tensor.to(target)
                                nv.requires_grad_(tensor.requires_grad)
                            moved_cache[id(tensor)] = nv
                        replacement = moved_cache[id(tensor)]
                    moves.append((m, name, tensor, replacement))
        snapshots = {}
        with _no_grad():
            for _, kind, _, current, value in staged:
                relocating = target is not None and current.device != target
                if kind == "parameter":
                    snapshots[id(current)] = (current.to(current.device), current._model_value_reference() if relocating else None)
                if kind == "buffer" or relocating:
                    value.requires_grad_(current.requires_grad)
        done = []

        def commit():
            with _no_grad():
                for owner, kind, name, current, value in staged:
                    done.append((owner, kind, name, current))
                    if kind == "buffer":
                        owner._set_member(name, value, "buffer", persistent=name not in owner._non_persistent_buffers)
                    elif target is not None and current.device != target:
                        current._rebind_model_value_(value)
                    else:
                        current._copy_data_(value)
                for owner, name, current, replacement in moves:
                    done.append((owner, "buffer", name, current))
                    owner._set_member(name, replacement, "buffer", persistent=name not in owner._non_persistent_buffers)

        def rollback():
            with _no_grad():
                for owner, kind, name, current in reversed(done):
                    if kind == "buffer":
                        owner._set_member(name, current, "buffer", persistent=name not in owner._non_persistent_buffers)
                    else:
                        values, representation = snapshots[id(current)]
                        if representation is not None:
                            current._rebind_model_value_(representation)
                        current._copy_data_(values)
                done.clear()

        def placement(parameter):
            return target if target is not None and id(parameter) in param_ids else parameter.device

        return PreparedLoad(commit, rollback, placement)

    # -------------------------------------------------------------------- call
    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)

    def forward(self, *args, **kwargs):
        raise NotImplementedError(f"{type(self).__name__} must implement forward()")

    def __repr__(self):
        name = type(self).__name__
        if not (self._modules or self._parameters or self._buffers):
            return f"{name}()"
        lines = [f"{name}("]
        lines += [f"  ({k}): {m!r}" for k, m in self._modules.items()]
        lines += [f"  ({k}): Parameter(shape={p.shape})" for k, p in self._parameters.items()]
        lines += [f"  ({k}): Buffer(shape={None if b is None else b.shape})" for k, b in self._buffers.items()]
        lines.append(")")
        return "\n".join(lines)
