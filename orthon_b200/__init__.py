"""orthon_b200: a Blackwell-native tensor and autograd runtime.

Public names follow the Orthon API (reference project: python/orthon/__init__.py:17-121):
tensors with views that share a versioned buffer, a frozen kernel registry behind every
operator, a reverse-mode engine with ``retain_graph``, ``nn`` modules, SGD/Adam, explicit AMP,
data-parallel training and pickle-free checkpoints.  The native extension is built in-tree by
``build.py``; importing the package without it raises immediately instead of falling back.
"""
from contextlib import contextmanager as _contextmanager

try:
    from . import _C
except ImportError as exc:  # pragma: no cover - build problem, never a silent fallback
    raise ImportError(
        "orthon_b200._C is not built; run `python build.py` at the repository root"
    ) from exc



def _check_build_matches_sources():
    """A checkout carries the native sources next to the package.  If they differ from the ones
    the extension was built from, Python code may call bindings that do not exist yet (or exist
    with another signature): refuse to import instead of failing somewhere inside a run."""
    import hashlib
    import os
    csrc = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
    built = getattr(_C, "_source_digest", None)
    if built is None or not os.path.isdir(csrc) or os.environ.get("ORTHON_SKIP_BUILD_CHECK") == "1":
        return
    h = hashlib.sha256()
    paths = []
    for root, _, files in os.walk(csrc):
        for name in files:
            if name.endswith((".cpp", ".cu", ".h", ".hpp", ".cuh")):
                full = os.path.join(root, name)
                paths.append((os.path.relpath(full, csrc).replace(os.sep, "/"), full))
    for rel, full in sorted(paths):
        h.update(rel.encode())
        h.update(b"\0")
        with open(full, "rb") as f:
            h.update(f.read())
    if h.hexdigest() != built:
        raise ImportError("orthon_b200._C was built from other sources than the ones under csrc/ "
                          "(stale extension); run `python build.py` at the repository root")


_check_build_matches_sources()

from ._C import (  # noqa: F401,E402
    DType, DeviceType, Device, Tensor, UnsupportedOperation,
    isfinite_all, empty, zeros, ones, full, from_numpy, fill_,
    add, mul, sub, div, reshape, transpose, contiguous,
    sum, mean, max, argmax,
    neg, relu, sigmoid, tanh, leaky_relu, gelu, exp, log, sqrt, reciprocal,
    dropout, embedding, to, cast, matmul, linear, fused_linear_relu,
    cuda_enabled, cuda_available, cuda_device_count, cuda_synchronize,
    set_float32_matmul_precision, get_float32_matmul_precision,
    is_grad_enabled, set_grad_enabled,
    softmax, log_softmax, cross_entropy, nll_loss, conv2d, maxpool2d,
    _amp_unscale_to_float32_and_check, _amp_copy_master_to_model_,
    _tensor_to_bytes, _tensor_from_bytes,
)

nccl_enabled = _C.nccl_enabled


def flatten(tensor, start_dim=0, end_dim=-1):
    return tensor.flatten(start_dim, end_dim)


def layer_norm(tensor, normalized_shape, weight=None, bias=None, eps=1e-5):
    from .functional import layer_norm as _impl
    return _impl(tensor, normalized_shape, weight=weight, bias=bias, eps=eps)


def scaled_dot_product_attention(q, k, v, mask=None, dropout_p=0.0, training=True, is_causal=False):
    from .functional import scaled_dot_product_attention as _impl
    return _impl(q, k, v, mask=mask, dropout_p=dropout_p, training=training, is_causal=is_causal)


@_contextmanager
def no_grad():
    previous = is_grad_enabled()
    set_grad_enabled(False)
    try:
        yield
    finally:
        set_grad_enabled(previous)


from ._random import manual_seed  # noqa: E402,F401
from . import functional, nn, optim, amp, training  # noqa: E402,F401
from .checkpoint import (  # noqa: E402,F401
    save_state_dict, load_state_dict, save_checkpoint, load_checkpoint,
)
from . import distributed  # noqa: E402,F401

__version__ = "0.1.0"
