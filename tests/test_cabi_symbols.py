"""The C-ABI library loads without a GPU and exports every function include/b200llm.h declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "b200llm.h")


def declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    names = re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", src)
    return sorted(set(names))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for must in ("b200_store_kvcache", "b200_paged_decode_gqa", "b200_prefill_varlen", "b200_mla_decode",
                 "b200_block_hash", "b200_abi_version"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from llm_from_scratch_b200 import _build, _lib
    if not _lib.LIB_PATH.exists():
        _build.build()
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} declared in b200llm.h but not exported"
    assert set(_lib.SIGNATURES) == set(declared_functions())
    want = int(re.search(r"#define\s+B200_ABI_VERSION\s+(\d+)", open(HEADER).read()).group(1))
    assert _lib.lib.b200_abi_version() == want >= 9
    assert _lib.lib.b200_strerror(-3) == b"unsupported shape or dtype"


def test_argument_errors_are_reported_without_a_gpu():
    """Pure argument validation happens before any CUDA call."""
    from llm_from_scratch_b200._lib import lib
    assert lib.b200_store_kvcache(None, None, 0, 0, None, None, None, -1, 1, 1, 0, 0, None, None) == -1
    assert lib.b200_paged_decode_gqa(None, None, None, None, None, 0, None, 1, 7, 2, 64, 16, 1, 1.0,
                                     None, 0, 1, None, None) == -1  # 7 heads not divisible by 2
    assert lib.b200_prefill_varlen(None, None, None, None, 0, 0, 0, 1, 1, None, None, 1, 1, 1, 4, 4, 64, 64,
                                   1.0, None, None, None, 0, 0, 0, None, None, 0, 0, 5, None, None) == -3  # bad dtype
    assert lib.b200_prefill_tile_rows(32, 8, 128, 128, 1) == 256      # tcgen05 kernel, two row tiles per CTA
    assert lib.b200_prefill_tile_rows(16, 16, 192, 128, 1) == 256     # tcgen05 kernel, two row tiles per CTA
    assert lib.b200_prefill_tile_rows(16, 4, 64, 64, 1) == 128        # tcgen05 kernel, four heads of a KV head per CTA
    assert lib.b200_prefill_tile_rows(4, 2, 64, 64, 1) == 64          # group of two: mma.sync kernel
    assert lib.b200_prefill_tile_rows(16, 4, 64, 64, 0) == 0          # fp32: general kernel only
    assert lib.b200_prefill_plan_bytes(1000, 7, 64) == (4 + 16 + 7) * 4
    assert lib.b200_prefill_plan(None, 1, 10, 64, None, 0, None, None) == -1
    assert lib.b200_mla_decode(None, None, None, None, None, 0, None, 1, 16, 512, 64, 16, 1, 1.0,
                               None, 0, 1, None, None) == -1  # bt_stride 0


def test_xxh64_matches_the_oracle_on_random_lengths():
    import random
    from llm_from_scratch_b200._lib import lib
    from oracle.xxh64 import xxh64
    rng = random.Random(0)
    for n in list(range(0, 70)) + [255, 256, 1000]:
        data = bytes(rng.randrange(256) for _ in range(n))
        for seed in (0, 1, 2 ** 63 + 11):
            assert lib.b200_xxh64(data, n, seed) == xxh64(data, seed)
