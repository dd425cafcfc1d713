"""geoweave_b200 -- B200 (sm_100a) implementation of GeoWeave's sparse top-k global-attention path.

Three stages, each a hand-written CUDA kernel behind a C ABI (``include/geoweave_b200.h``):

1. indexer score ``sum_h w[s,h] * relu(scale * q_idx[t,h] . k_idx[s,h])`` on tcgen05 tensor cores,
2. exact per-query top-k fused into that kernel's epilogue (ties keep the lower key index),
3. sparse attention of each query over only its selected keys.

The sub-packages keep the call signatures of the reference's operator modules, so the reference's
``DSAAttention`` / ``LightningIndexer`` can use them unchanged:

* ``geoweave_b200.custom_indexer``      <->  ``easyvolcap.utils.custom_indexer``
* ``geoweave_b200.custom_flash_attn``   <->  ``easyvolcap.utils.custom_flash_attn``

``install()`` rebinds the reference's module-level names to these functions.  There is no CPU or Triton
fallback: every call needs the built library (``python -m geoweave_b200.build``) and a CUDA device.
"""
from __future__ import annotations

import importlib
import sys

from . import _lib
from ._lib import GeoWeaveError, check_status, clear_runtime_cache  # noqa: F401

__version__ = "0.1.0"

__all__ = ["install", "uninstall", "GeoWeaveError", "check_status", "clear_runtime_cache", "library_path"]

_saved: dict = {}

# (reference module, attribute) -> (our module, attribute).  The reference binds these names with
# `from ... import ...` inside try/except at import time (official_vggt/layers/indexer.py:10-14,
# official_vggt/layers/dsa_attention.py:29-44), so both the defining and the importing modules are patched.
_BINDINGS = [
    ("easyvolcap.utils.custom_indexer", "sparse_topk_indexer_func", "geoweave_b200.custom_indexer", "sparse_topk_indexer_func"),
    ("easyvolcap.utils.custom_indexer", "sparse_topk_indexer_inference_func", "geoweave_b200.custom_indexer", "sparse_topk_indexer_inference_func"),
    ("easyvolcap.official_vggt.layers.indexer", "sparse_topk_indexer_func", "geoweave_b200.custom_indexer", "sparse_topk_indexer_func"),
    ("easyvolcap.official_vggt.layers.indexer", "sparse_topk_indexer_inference_func", "geoweave_b200.custom_indexer", "sparse_topk_indexer_inference_func"),
] + [
    (mod, name, "geoweave_b200.custom_flash_attn", name)
    for mod in ("easyvolcap.utils.custom_flash_attn.sparse_index_flash_attn", "easyvolcap.official_vggt.layers.dsa_attention")
    for name in ("sparse_index_flash_attn_func", "sparse_index_flash_attn_bhtd_func", "dense_index_flash_attn_func",
                 "sparse_index_flash_attn_inference_func", "sparse_index_flash_attn_inference_bhtd_func",
                 "sparse_index_flash_attn_value_gate_bhtd_func")
]


def library_path() -> str:
    return _lib.LIB_PATH


def install(import_missing: bool = True) -> list:
    """Point the reference's operator names at this library.  Returns the list of patched ``module.attr``.

    The reference must be importable (``easyvolcap`` on ``sys.path``).  Modules that are not imported yet are
    imported first when ``import_missing`` is true.  Fails loudly if the CUDA library cannot be loaded.
    """
    _lib.load()
    patched = []
    for ref_mod, ref_attr, our_mod, our_attr in _BINDINGS:
        mod = sys.modules.get(ref_mod)
        if mod is None:
            if not import_missing:
                continue
            mod = importlib.import_module(ref_mod)
        ours = getattr(importlib.import_module(our_mod), our_attr)
        key = (ref_mod, ref_attr)
        if key not in _saved:
            _saved[key] = getattr(mod, ref_attr, None)
        setattr(mod, ref_attr, ours)
        patched.append(f"{ref_mod}.{ref_attr}")
    return patched


def uninstall() -> None:
    """Undo ``install()``."""
    for (ref_mod, ref_attr), old in _saved.items():
        mod = sys.modules.get(ref_mod)
        if mod is not None:
            setattr(mod, ref_attr, old)
    _saved.clear()
