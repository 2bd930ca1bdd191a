"""ctypes binding of ``libb200llm.so`` (the C ABI declared in ``include/b200llm.h``).

There is no fallback: if the library has not been built, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libb200llm.so"

DTYPE_F32 = 0
DTYPE_BF16 = 1

ERR_BOUNDS = -6

_vp, _i32, _i64, _f32, _sz, _u64 = C.c_void_p, C.c_int32, C.c_int64, C.c_float, C.c_size_t, C.c_uint64

# name -> (restype, argtypes); mirrors include/b200llm.h declaration by declaration
SIGNATURES = {
    "b200_abi_version": (_i32, []),
    "b200_strerror": (C.c_char_p, [_i32]),
    "b200_sm_count": (_i32, []),
    "b200_read_status": (_i32, [_vp, _vp, _vp]),
    "b200_xxh64": (_u64, [_vp, _sz, _u64]),
    "b200_block_hash": (_u64, [_vp, _i32, _u64, _i32]),
    "b200_block_hash_chain": (_i64, [_vp, _i64, _i32, _vp]),
    "b200_pool_create": (_vp, [_i64, _i32]),
    "b200_pool_destroy": (None, [_vp]),
    "b200_pool_num_free": (_i64, [_vp]),
    "b200_pool_allocate": (_i64, [_vp, _vp, _i64, _vp, _vp]),
    "b200_pool_deallocate": (_i32, [_vp, _vp, _i64]),
    "b200_pool_append": (_i64, [_vp, _i32, _i32, _i64, _vp]),
    "b200_pool_open_block": (_i64, [_vp]),
    "b200_pool_seal_block": (_i32, [_vp, _i32, _i32, _vp]),
    "b200_pool_lookup": (_i64, [_vp, _u64]),
    "b200_pool_snapshot": (_i64, [_vp, _vp, _vp, _vp, _vp]),
    "b200_prepare_prefill": (_i64, [_i32, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _i64, _vp]),
    "b200_prepare_decode": (_i32, [_i32, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _i64]),
    "b200_store_kvcache": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp, _vp, _i32, _i32, _i32, _i64,
                                  _i32, _vp, _vp]),
    "b200_paged_decode_gqa_workspace_bytes": (_sz, [_i32, _i32, _i32, _i32, _i32]),
    "b200_paged_decode_gqa": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _vp, _i32, _i32, _i32, _i32,
                                     _i32, _i64, _f32, _vp, _sz, _i32, _vp, _vp]),
    "b200_paged_decode_gqa_static": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _vp, _i32, _i32, _i32,
                                            _i32, _i32, _i64, _f32, _i32, _vp, _vp]),
    "b200_prefill_varlen_shared_tail": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _vp, _vp, _i32, _i32,
                                               _i32, _i32, _i32, _i32, _f32, _vp, _i32, _i32, _i32, _vp, _vp]),
    "b200_prefill_varlen": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _vp, _i32, _i32,
                                   _i32, _i32, _i32, _i32, _i32, _f32, _vp, _vp, _vp, _i64, _i32,
                                   _i64, _vp, _vp, _i32, _i32, _i32, _vp, _vp]),
    "b200_prefill_tile_rows": (_i32, [_i32, _i32, _i32, _i32, _i32]),
    "b200_prefill_plan_bytes": (_sz, [_i64, _i32, _i32]),
    "b200_prefill_plan": (_i32, [_vp, _i32, _i32, _i32, _vp, _sz, _vp, _vp]),
    "b200_add_rmsnorm": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _f32, _i32, _i32, _vp]),
    "b200_mla_prologue": (_i32, [_vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _i64, _i64,
                                 _i32, _i32, _i32, _i32, _f32, _i32, _vp, _vp]),
    "b200_qk_norm_rope_store": (_i32, [_vp, _i64, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64,
                                       _i32, _i32, _i32, _f32, _i32, _vp, _vp]),
    "b200_moe_route_workspace_bytes": (_sz, [_i32, _i32]),
    "b200_moe_route": (_i32, [_vp, _vp, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _sz, _i32, _vp]),
    "b200_moe_gate_route_workspace_bytes": (_sz, []),
    "b200_moe_gate_route": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _vp,
                                   _sz, _i32, _vp]),
    "b200_swiglu": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32, _i32, _vp]),
    "b200_moe_grouped_gemm": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp]),
    "b200_decode_advance": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _i64, _i32, _vp, _vp, _vp]),
    "b200_block_table_patch": (_i32, [_vp, _i32, _vp, _i64, _i32, _vp, _vp]),
    "b200_sample": (_i32, [_vp, _i64, _vp, _i64, _i32, _u64, _u64, _vp, _i32, _vp]),
    "b200_moe_combine": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _vp]),
    "b200_selftest_bounded_wait": (_i32, [_i32, _vp, _vp, _vp]),
    "b200_lm_head_argmax_workspace_bytes": (_sz, [_i32, _i32]),
    "b200_lm_head_argmax": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp, _sz, _i32, _vp, _vp]),
    "b200_mla_decode_workspace_bytes": (_sz, [_i32, _i32, _i32, _i32, _i32]),
    "b200_mla_decode": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _vp, _i32, _i32, _i32, _i32, _i32,
                               _i64, _f32, _vp, _sz, _i32, _vp, _vp]),
}


def load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build the CUDA library first "
            "(python -m llm_from_scratch_b200._build); there is no CPU fallback")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = load()


class B200Error(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise B200Error(f"{what}: {lib.b200_strerror(rc).decode()} ({rc})")
