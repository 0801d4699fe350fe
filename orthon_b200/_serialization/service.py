"""Save / load orchestration.  Loading decodes and validates the WHOLE archive first, then
prepares the model, then the optimizer (told where the model's parameters will live), and only
then commits, model first, with reverse rollback on failure.
(reference project: python/orthon/_serialization/service.py:44-82, transaction.py:23-84)"""
from .. import _C
from .archive import Archive, fspath, write_archive
from .codec import Decoder, Encoder
from .format import FORMAT_ID, FORMAT_VERSION, fail
from .transaction import RestoreTransaction


def _device(spec, api):
    if spec is None or isinstance(spec, _C.Device):
        return spec
    if isinstance(spec, str):
        try:
            return _C.Device(spec)
        except Exception as exc:  # noqa: BLE001
            raise ValueError(f"{api}: unknown map_location {spec!r} ({exc})") from None
    raise TypeError(f"{api}: map_location must be a device string or Device, got {type(spec)!r}")


def save_checkpoint(path, model=None, optimizer=None, metadata=None):
    target = fspath(path, "save_checkpoint")
    enc = Encoder()
    model_section = None
    if model is not None:
        if not hasattr(model, "state_dict"):
            raise TypeError("save_checkpoint: model must expose state_dict()")
        state = model.state_dict()
        items = []
        for name in sorted(state):  # sorted in the file only
            if not isinstance(state[name], _C.Tensor):
                raise TypeError(f"save_checkpoint: model state entry {name!r} must be a Tensor, got {type(state[name])!r}")
            items.append([name, enc.encode(state[name], f"model.{name}")])
        model_section = {"k": "dict", "v": items}
    optimizer_section = None
    if optimizer is not None:
        if not hasattr(optimizer, "state_dict"):
            raise TypeError("save_checkpoint: optimizer must expose state_dict()")
        optimizer_section = enc.encode(optimizer.state_dict(), "optimizer")
    metadata_section = enc.encode(dict(metadata or {}), "metadata")
    manifest = {"format": FORMAT_ID, "format_version": FORMAT_VERSION,
                "sections": {"model": model_section, "optimizer": optimizer_section, "metadata": metadata_section}}
    write_archive(target, manifest, enc.payloads)


def load_checkpoint(path, model=None, optimizer=None, map_location=None):
    target = _device(map_location, "load_checkpoint")
    with Archive(path) as archive:
        sections = archive.read_manifest()
        dec = Decoder(archive.read_payload)
        restored = {}
        for name in ("model", "optimizer", "metadata"):
            node = sections[name]
            restored[name] = None if (node is None and name != "metadata") else dec.decode(node, name)
        ms = restored["model"]
        if sections["model"] is not None and (not isinstance(ms, dict) or not all(
                isinstance(k, str) and isinstance(v, _C.Tensor) for k, v in ms.items())):
            fail("model section is not a Tensor state mapping")
        if not isinstance(restored["metadata"], dict):
            fail("metadata section is not a mapping")
    if model is not None and sections["model"] is None:
        fail("checkpoint has no model section")
    if optimizer is not None and sections["optimizer"] is None:
        fail("checkpoint has no optimizer section")
    RestoreTransaction.prepare(model, ms, optimizer, restored["optimizer"], map_location=target).commit()
    return restored["metadata"]


class SerializationService:
    """Object form of the two entry points (what `checkpoint.save_checkpoint` / `load_checkpoint`
    delegate to); kept separate from the codec and the archive so either can be replaced."""

    save = staticmethod(save_checkpoint)
    load = staticmethod(load_checkpoint)
