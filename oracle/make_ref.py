"""Recipe for `oracle/_ref/`: the reference's OWN PyTorch implementation, staged so that the
benchmark's CPU baseline can time it on the GPU box's host cores.  TEST INFRASTRUCTURE - the
shipped package never imports anything from here.

The reference is pure Python.  Installing it with pip into a target folder fails offline (its
build backend, hatchling, is not available), so `stage()` copies the package directory
`lookahead_keys_attention/` as it lies in the reference checkout into `oracle/_ref/`.  That
folder is git-ignored: the reference's sources never enter this repository's history; like the
built `.so` they only travel with a snapshot of the working tree.  `__graft_entry__.build()` runs
`stage()` wherever the reference checkout exists.

The reference imports the third-party `rotary_embedding_torch` at module level
(lookahead_keys_attention/lookahead_keys_attention.py:13), which is not installed here.  No
configuration that is timed enables rotary embeddings, so `load_reference()` registers an empty
stand-in module of that name (never instantiated) before importing, exactly as
`tests/golden/make_golden.py` does when it records the golden vectors.

    python oracle/make_ref.py [/path/to/reference]      # stage by hand
"""
from __future__ import annotations

import shutil
import sys
import types
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_DIR = HERE / "_ref"
DEFAULT_CHECKOUT = Path("/root/reference")
PACKAGE = "lookahead_keys_attention"


def stage(checkout: Path | str = DEFAULT_CHECKOUT) -> Path | None:
    """Copy the reference package into oracle/_ref/.  Returns the folder, or None when the
    checkout is absent (the already staged copy, if any, is then left as it is)."""
    src = Path(checkout) / PACKAGE
    if not src.is_dir():
        return REF_DIR if available() else None
    dst = REF_DIR / PACKAGE
    if dst.exists():
        shutil.rmtree(dst)
    REF_DIR.mkdir(exist_ok=True)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__"))
    (REF_DIR / "STAGED_FROM").write_text(f"{src}\n")
    return REF_DIR


def available() -> bool:
    return (REF_DIR / PACKAGE / "lookahead_keys_attention.py").is_file()


def load_reference():
    """The reference's `Castle` class from the staged copy (PyTorch path; use_triton=False)."""
    if not available():
        raise RuntimeError("oracle/_ref is not staged; run oracle/make_ref.py where the reference checkout exists")
    try:
        import rotary_embedding_torch  # noqa: F401
    except ImportError:
        stub = types.ModuleType("rotary_embedding_torch")
        stub.RotaryEmbedding = object
        sys.modules["rotary_embedding_torch"] = stub
    if str(REF_DIR) not in sys.path:
        sys.path.insert(0, str(REF_DIR))
    from lookahead_keys_attention.lookahead_keys_attention import Castle
    return Castle


if __name__ == "__main__":
    out = stage(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_CHECKOUT)
    print(f"staged: {out}" if out else "reference checkout not found; nothing staged")
