"""ZIP + JSON container IO: deterministic writer with atomic replace, strict reader.

Writer: ``manifest.json`` deflated (sorted keys, compact separators, no NaN literals),
tensor payloads STORED, fixed timestamps and attributes, temp file in the destination
directory + fsync + ``os.replace``.  Reader: identifies files by content, refuses pickle
streams by header, rejects duplicate member names, duplicate JSON fields at any depth, bare
NaN/Infinity literals, compressed or mis-sized payloads.
(reference project: python/orthon/_serialization/archive.py:74-232)"""
import json
import os
import tempfile
import zipfile

from .format import (FORMAT_ID, FORMAT_VERSION, MANIFEST_NAME, MAX_JSON_DEPTH, MAX_MANIFEST_BYTES, PAYLOAD_RE,
                     ZIP_DATE_TIME, ZIP_EXTERNAL_ATTR, fail)


def fspath(path, api):
    try:
        p = os.fspath(path)
    except TypeError:
        raise TypeError(f"{api}: path must be str or os.PathLike, got {type(path)!r}") from None
    if isinstance(p, bytes):
        p = os.fsdecode(p)
    return p


def _member(name, compress):
    info = zipfile.ZipInfo(name, date_time=ZIP_DATE_TIME)
    info.compress_type = compress
    info.external_attr = ZIP_EXTERNAL_ATTR
    info.create_system = 0
    return info


def write_archive(target, manifest, payloads):
    """`payloads` is an ordered list of (member name, bytes)."""
    text = json.dumps(manifest, sort_keys=True, separators=(",", ":"), allow_nan=False, ensure_ascii=True)
    blob = text.encode("utf-8")
    if len(blob) > MAX_MANIFEST_BYTES:
        fail("manifest exceeds the size limit")
    directory = os.path.dirname(os.path.abspath(target))
    if not os.path.isdir(directory):
        raise FileNotFoundError(f"save_checkpoint: directory does not exist: {directory}")
    fd, tmp = tempfile.mkstemp(prefix=".ckpt-", suffix=".tmp", dir=directory)
    try:
        with os.fdopen(fd, "wb") as handle:
            with zipfile.ZipFile(handle, "w", allowZip64=True) as zf:
                zf.writestr(_member(MANIFEST_NAME, zipfile.ZIP_DEFLATED), blob)
                for name, data in payloads:
                    zf.writestr(_member(name, zipfile.ZIP_STORED), data)
            handle.flush()
            os.fsync(handle.fileno())
        os.replace(tmp, target)
    except BaseException:
        try:
            os.unlink(tmp)
        except OSError:
            pass
        raise


def _no_duplicate_pairs(pairs):
    out = {}
    for key, value in pairs:
        if key in out:
            fail(f"duplicate JSON field {key!r}")
        out[key] = value
    return out


def _reject_constant(token):
    fail(f"non-standard JSON literal {token}")


def _depth(value, limit=MAX_JSON_DEPTH):
    stack = [(value, 1)]
    while stack:
        node, d = stack.pop()
        if d > limit:
            fail("manifest nesting is too deep")
        if isinstance(node, dict):
            stack.extend((v, d + 1) for v in node.values())
        elif isinstance(node, list):
            stack.extend((v, d + 1) for v in node)


class Archive:
    def __init__(self, path, api="load_checkpoint"):
        self._path = fspath(path, api)
        self._zip = None

    def __enter__(self):
        with open(self._path, "rb") as f:
            head = f.read(4)
        if head[:1] == b"\x80":
            fail("file is a pickle stream; pickle checkpoints are refused without being read")
        if head[:2] != b"PK":
            fail("file is not a checkpoint archive")
        try:
            self._zip = zipfile.ZipFile(self._path, "r")
        except zipfile.BadZipFile as exc:
            fail(f"corrupt archive ({exc})")
        names = [i.filename for i in self._zip.infolist()]
        if len(names) != len(set(names)):
            self._zip.close()
            fail("duplicate archive member names")
        return self

    def __exit__(self, *exc):
        if self._zip is not None:
            self._zip.close()
        return False

    def read_manifest(self):
        try:
            info = self._zip.getinfo(MANIFEST_NAME)
        except KeyError:
            fail("manifest.json is missing")
        if info.file_size > MAX_MANIFEST_BYTES:
            fail("manifest exceeds the size limit")
        raw = self._zip.read(info)
        try:
            text = raw.decode("utf-8")
            try:
                manifest = json.loads(text, object_pairs_hook=_no_duplicate_pairs, parse_constant=_reject_constant)
            except RecursionError:
                fail("manifest nesting is too deep")
        except UnicodeDecodeError:
            fail("manifest is not UTF-8")
        except json.JSONDecodeError as exc:
            fail(f"manifest is not valid JSON ({exc.msg})")
        _depth(manifest)
        if not isinstance(manifest, dict) or manifest.get("format") != FORMAT_ID:
            fail("unknown container format")
        version = manifest.get("format_version")
        if type(version) is not int or version != FORMAT_VERSION:
            fail(f"unsupported format_version {version!r}")
        sections = manifest.get("sections")
        if not isinstance(sections, dict) or set(sections) != {"model", "optimizer", "metadata"}:
            fail("manifest sections are malformed")
        return sections

    def read_payload(self, name, nbytes, where):
        if not isinstance(name, str) or not PAYLOAD_RE.match(name):
            fail(f"{where}: invalid payload name {name!r}")
        try:
            info = self._zip.getinfo(name)
        except KeyError:
            fail(f"{where}: payload {name} is missing")
        if info.compress_type != zipfile.ZIP_STORED:
            fail(f"{where}: payload {name} must be stored uncompressed")
        if info.file_size != nbytes or info.compress_size != nbytes:
            fail(f"{where}: payload {name} has {info.file_size} bytes, expected {nbytes}")
        data = self._zip.read(info)
        if len(data) != nbytes:
            fail(f"{where}: payload {name} is truncated")
        return data
