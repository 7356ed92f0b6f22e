"""Load the unmodified reference (nilesh2797/BlockRank) from ``baseline/_ref`` for comparison runs.

``baseline/_ref`` is produced by ``baseline/install_ref.sh`` (an offline ``pip install --target`` of the
reference checkout); it is not tracked by git.  ``import blockrank`` does not work in this image: the
package ``__init__`` imports training-only dependencies (pytrec_eval, trl, peft) that are absent.  The
files on the prefill path need only torch / transformers / triton, so they are loaded by file path:

    src/blockrank/blockrank_std_attention.py          eager / sdpa BlockRank attention + mask builder
    src/blockrank/blockrank_triton_kernel_attention.py  the Triton kernels (GPU only)
    src/blockrank/losses.py                            compute_auxiliary_attention_loss

transformers >= 5 calls mask functions without ``cache_position``; ``mask_shim`` supplies it, nothing
else of the reference is altered.  Used by ``bench.py --impl reference``, the ``cpu_baseline`` leg and
``opbench.py``; never by the product path.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF_PKG = os.path.join(HERE, "_ref", "blockrank")
FILES = {"std": "blockrank_std_attention.py", "triton": "blockrank_triton_kernel_attention.py",
         "losses": "losses.py"}


def available() -> bool:
    return all(os.path.exists(os.path.join(REF_PKG, f)) for f in FILES.values())


def why_unavailable() -> str:
    return (f"{REF_PKG} is missing: run baseline/install_ref.sh where the reference checkout is available "
            "(the installed copy travels to the GPU box with the working tree)")


_cache = {}


def load(which: str) -> types.ModuleType:
    """which in {'std', 'triton', 'losses'} -> the reference module, loaded by path (cached)."""
    if which in _cache:
        return _cache[which]
    if not available():
        raise ImportError(why_unavailable())
    name = "blockrank_ref_" + which
    spec = importlib.util.spec_from_file_location(name, os.path.join(REF_PKG, FILES[which]))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    _cache[which] = mod
    return mod


def mask_shim(mask_fn):
    """Adapt a reference mask function (batch_size, cache_position, kv_length, ...) to the keyword-only
    call transformers >= 5 makes (batch_size, q_length, kv_length, q_offset, kv_offset, ...)."""
    def shim(*a, **kw):
        kw.pop("q_length", None)
        kw.pop("q_offset", None)
        if a:
            return mask_fn(*a, **kw)
        return mask_fn(kw.pop("batch_size"), kw.pop("cache_position", None), kw.pop("kv_length"), **kw)
    return shim


def register(name: str = "eager_blockrank") -> str:
    """Register the reference's attention + mask functions in the transformers registries under ``name``
    (one of eager_blockrank, sdpa_blockrank, triton_blockrank), with the calling-convention shim."""
    from transformers import AttentionInterface, AttentionMaskInterface
    if name == "triton_blockrank":
        tri = load("triton")
        AttentionInterface.register(name, tri.triton_blockrank_attention_forward)
        AttentionMaskInterface.register(name, mask_shim(tri.triton_blockrank_attention_mask))
        return name
    std = load("std")
    fwd = {"eager_blockrank": std.eager_blockrank_attention_forward,
           "sdpa_blockrank": std.sdpa_blockrank_attention_forward}[name]
    AttentionInterface.register(name, fwd)
    AttentionMaskInterface.register(name, mask_shim(std.eager_blockrank_attention_mask))
    return name


class AttnModule:
    """The attributes of an HF attention module the reference functions read."""

    def __init__(self, groups: int, layer_idx: int = 0):
        self.num_key_value_groups = groups
        self.layer_idx = layer_idx
        self.training = False
