"""Loads the compiled kernel libraries and declares their C signatures.

There is no fallback: if a library cannot be compiled or loaded, or no CUDA device is present, the
first kernel call raises ``KernelsUnavailable`` with the reason.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_void_p

from . import build as _build


class KernelsUnavailable(RuntimeError):
    pass


P, I, F, L = c_void_p, c_int, c_float, ctypes.c_longlong

# module -> {function: argument types}; every function returns an int (0, or a CUDA error code,
# or a negative number for arguments the kernel refuses)
SIGNATURES: dict[str, dict[str, list]] = {
    "core": {
        "de_embed_rows": [I, P, P, P, I, I, I, F, P],
        "de_add_rmsnorm": [I, I, P, P, P, P, P, I, I, F, P],
        "de_add_rmsnorm_grouped": [I, I, P, P, P, P, P, I, I, I, F, P],
        "de_rope_kv_write": [I, P, I, P, P, P, I, I, I, I, P, P, P, I, I, I, I, I, P, P],
        "de_silu_mul": [I, P, P, I, I, P],
        "de_sample_rows": [P, I, I, P, P, P, P, P],
        "de_add_layernorm": [I, I, P, P, P, P, P, P, I, I, F, P],
        "de_activation": [I, P, I, P, I, I, I, I, P],
        "de_softcap": [P, L, F, P],
        "de_scaled_sum": [I, P, P, F, F, P, L, P],
        "de_residual_add": [P, I, P, I, P, P, I, P, L, P],
        "de_act_mul": [I, P, I, P, I, I, I, I, P],
        "de_act_mul_row": [I, P, I, P, P, I, P, I, I, I, I, P],
        "de_add_normed": [I, I, P, P, P, I, I, F, P],
        "de_rmsnorm_cols": [I, I, P, I, P, P, I, I, I, F, P],
    },
    "gemm_f32": {
        "de_gemm_f32": [P, P, P, I, I, I, I, I, I, P], "de_gemm_f32_small_rows": [],
    },
    "attention_simt": {
        "de_attn_simt_rows_per_tile": [],
        "de_attn_simt": [I, P, I, P, I, P, P, P, I, I, P, P, P, P, P, I, P, P, I, I, I, I, F, I, P,
                         P],
        "de_attn_combine": [I, P, I, P, P, P, I, P, P, I, I, I, I, P],
    },
    "linear_small": {
        "de_linear_small_max_rows": [],
        "de_linear_small": [P, I, P, I, P, I, I, I, I, I, I, I, P],
        "de_linear_small_parts": [I],
        "de_linear_small_norm": [P, I, P, I, P, I, I, I, I, I, P, I, I, F, P, I, P, P, P],
    },
    "linear_mid": {
        "de_linear_mid_max_rows": [], "de_linear_mid_parts": [I],
        "de_linear_mid": [P, I, P, I, P, I, I, I, I, I, I, P, I, I, F, P, I, P, P, I, P, P],
    },
    "gemm_tcgen05": {
        "de_gemm_tcgen05": [P, I, P, I, P, I, I, I, I, I, I, P, P],
        "de_gemm_tcgen05_tile": [I, I, I], "de_gemm_tcgen05_sms": [],
        "de_gemm_tcgen05_grouped": [P, I, P, P, I, P, P, I, I, I, I, I, I, P, P],
    },
    "attention_tcgen05": {
        "de_attn_tcgen05_rows": [], "de_attn_tcgen05_head_dim": [],
        "de_attn_tcgen05": [P, I, P, I, P, P, P, I, I, P, P, P, P, P, I, P, P, I, I, I, I, F, I, P, P],
    },
    "attention_mma": {
        "de_attn_mma_head_dim": [], "de_attn_mma_rows": [I],
        "de_attn_mma": [I, P, I, P, I, P, P, P, I, I, P, P, P, P, P, I, P, P, I, I, I, I, F, I, P,
                        P],
    },
    "attention_chunk": {
        "de_attn_chunk_rows": [I, I, I, I],
        "de_attn_chunk_decode_ok": [I, I, I, I, I, I],
        "de_attn_chunk_decode": [I, P, I, P, I, P, P, P, I, I, P, P, P, I, P, P, I, I, I, I, I, F,
                                 I, I, I, F, I, I, P, I, P, I, P, I, I, I, P, P, I, I, P, P],
        "de_kv_write_rotated": [I, P, I, P, P, P, I, P, I, I, I, I, P, P, P, I, I, I, I, I, P, P],
        "de_attn_finish": [I, P, P, P, P, I, P, I, I, I, I, P],
        "de_conv_keep": [I, P, I, P, L, I, P, P, P, I, I, I, P],
        "de_qkv_prepare": [I, P, I, P, P, P, P, P, P, P, I, P, L, I, I, P, P, F, P, I, F, I, F, I,
                           I, P, P, I, I, I, I, I, P, P, P, I, I, I, I, P, P],
        "de_kv_write_normed": [I, P, I, I, P, P, I, I, I, F, P, P, P, I, I, I, I, P, P],
        "de_attn_chunk": [I, P, I, P, I, P, P, P, I, I, P, P, P, P, P, I, P, P, I, I, I, I, I, F,
                          I, I, I, F, I, I, I, I, P, P, I, I, P, P],
    },
    "recurrent": {
        "de_recurrent_max_key_dim": [],
        "de_delta_prep": [I, P, I, P, P, P, P, P, L, I, P, P, P, P, P, P, P, P, P, I, I, I, I, I,
                          I, I, P],
        "de_conv_state": [I, P, I, P, L, I, P, P, P, I, I, I, P],
        "de_retention_prep": [I, P, I, P, P, I, I, I, P, P, I, P],
        "de_state_scan": [I, I, P, I, P, I, P, I, P, I, P, I, P, I, P, P, L, P, P, P, P, I, I, I,
                          I, I, P, I, I, I, I, I, P],
        "de_gdelta_prep": [I, P, I, I, I, I, P, P, P, P, P, P, P, P, I, I, I, P],
        "de_silu_rows": [I, P, I, P, I, I, P],
        "de_head_gate": [I, P, P, I, P, P, I, I, I, F, I, P],
        "de_mean_of_normed": [I, P, P, P, P, P, I, I, F, P],
    },
    "latent": {
        "de_latent_write": [I, I, P, I, P, I, P, I, P, P, P, F, P, F, I, I, I, I, P, P, I, I, I, I,
                            P, P],
        "de_heads_product": [I, I, I, P, I, I, P, P, I, I, P, I, I, I, I, I, P],
    },
    "experts": {
        "de_experts_tiles": [I, I, I, I],
        "de_experts_gather": [I, P, I, P, I, I, I, P, P],
        "de_experts_route": [I, P, I, P, P, I, I, I, I, I, P, P, P],
        "de_experts_group": [P, I, I, I, I, P, P, P, P],
        "de_experts_up": [I, P, I, P, P, P, I, I, I, I, P, I, P],
        "de_experts_down": [I, P, P, P, P, I, I, I, P, P],
        "de_experts_combine": [I, P, P, I, I, I, P, P, I, P, I, P],
    },
    "sublayer": {
        "de_norm_stream": [I, I, P, P, P, I, I, F, P],
        "de_gated_normed_add": [I, I, I, P, P, I, P, P, P, P, P, I, I, F, P],
        "de_depth_mix": [I, P, L, P, I, L, P, P, P],
        "de_poly_norm": [I, P, I, P, P, I, I, I, F, P],
    },
    "attention_decode": {
        "de_attn_decode_head_dim": [], "de_attn_decode_max_cluster": [],
        "de_attn_decode_blocks_per_sm": [I],
        "de_attn_decode": [P, I, P, I, P, P, P, I, I, P, P, P, P, I, I, I, P, P, P, P, I, I, I, I,
                           I, I, F, I, P, P],
    },
}

_loaded: dict[tuple[str, tuple[str, ...]], ctypes.CDLL] = {}

# percent of an SM's memory that the decode step's kernels ask for as shared memory (-1: each
# kernel's default)
CARVEOUT = int(os.environ.get("DISTENGINE_B200_CARVEOUT", "50"))
CARVEOUT_MODULES = ("core", "linear_small", "attention_decode")


def default_build_requests() -> list[tuple[str, tuple[str, ...]]]:
    """Every module; the per-head-size attention for the head sizes of common models."""
    requests = [(module, ()) for module in _build.MODULES
                if module in SIGNATURES
                and module not in ("attention_mma", "attention_decode", "attention_tcgen05")]
    # (16: the head size of the tiny model that the smoke test generates with)
    return (requests + [("attention_mma", (f"HEAD_DIM={d}",)) for d in (16, 64, 128)]
            + [("attention_tcgen05", (f"HEAD_DIM={d}",)) for d in (64, 128)]
            + [("attention_decode", (f"HEAD_DIM={d}",)) for d in (16, 64, 128)])


def load(module: str, defines: tuple[str, ...] = ()) -> ctypes.CDLL:
    key = (module, defines)
    lib = _loaded.get(key)
    if lib is not None:
        return lib
    try:
        path = _build.build(module, defines)
        lib = ctypes.CDLL(path)
    except (_build.BuildError, OSError) as error:
        raise KernelsUnavailable(
            f"the CUDA kernel library '{module}' of distengine_b200 could not be built or "
            f"loaded: {error}") from error
    for name, argtypes in SIGNATURES[module].items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int
    # programmatic dependent launch (a kernel may start while the one before it finishes) is on
    # unless DISTENGINE_B200_PDL=0
    lib.de_set_pdl.argtypes = [c_int]
    lib.de_set_pdl.restype = c_int
    lib.de_set_pdl(0 if os.environ.get("DISTENGINE_B200_PDL", "1") == "0" else 1)
    # the kernels of a decode step ask for one split of an SM's memory (see csrc/common.cuh)
    if module in CARVEOUT_MODULES:
        lib.de_set_carveout.argtypes = [c_int]
        lib.de_set_carveout.restype = c_int
        lib.de_set_carveout(CARVEOUT)
    _loaded[key] = lib
    return lib


def preload(modules: list[tuple[str, tuple[str, ...]]]) -> None:
    """Compile several modules side by side, then load them."""
    missing = [m for m in modules if m not in _loaded]
    if missing:
        try:
            _build.build_many(missing)
        except _build.BuildError as error:
            raise KernelsUnavailable(str(error)) from error
    for module, defines in modules:
        load(module, defines)
