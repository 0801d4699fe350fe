"""Wire constants of the v1 container and the uniform integrity error.
(reference project: python/orthon/_serialization/format.py:4-34)"""
import re

FORMAT_ID = "ml-runtime-checkpoint"
FORMAT_VERSION = 1
MANIFEST_NAME = "manifest.json"
PAYLOAD_RE = re.compile(r"^tensors/[0-9]{6}\.bin$")
ZIP_DATE_TIME = (1980, 1, 1, 0, 0, 0)   # fixed so equal states give equal bytes
ZIP_EXTERNAL_ATTR = 0o600 << 16
MAX_MANIFEST_BYTES = 8 << 20
MAX_JSON_DEPTH = 128


def fail(message):
    raise RuntimeError("checkpoint: " + message)
