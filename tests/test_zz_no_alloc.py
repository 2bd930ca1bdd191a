"""The allocation-free paged-decode entry point, called straight through the C ABI.

Who needs it: a host that has given every byte of device memory to its KV pool, or that is not
allowed to call an allocator while a decode step is in flight, cannot hand the kernel a scratch
buffer.  ``b200_paged_decode_gqa_static`` keeps the split-context scratch in a fixed 8 MiB device
array inside the library instead.  These tests check that it returns what the ordinary entry
point returns (same tolerance as the other bf16 parity tests), on two calls in a row with
different batches so that whatever the first call left in the shared array cannot leak into the
second, and that a problem too large for the array is refused rather than allocated for.

This file is named so that pytest collects it last.
"""
import numpy as np
import pytest
import torch

from llm_from_scratch_b200.workloads import deal_blocks

pytestmark = pytest.mark.gpu

BF16_MAX_ABS = 2e-2
ERR_TOO_LARGE = -8


def _case(lens, Hq, Hkv, D, seed):
    g = torch.Generator().manual_seed(seed)
    case = deal_blocks(lens, 16, np.random.default_rng(seed), pad_blocks=1)
    q = torch.randn(len(lens), Hq, D, generator=g).to(torch.bfloat16).cuda()
    kc = torch.randn(case.num_blocks, 16, Hkv, D, generator=g).to(torch.bfloat16).cuda()
    vc = torch.randn(case.num_blocks, 16, Hkv, D, generator=g).to(torch.bfloat16).cuda()
    bt = torch.from_numpy(case.block_tables).cuda()
    cl = torch.from_numpy(case.context_lens).cuda()
    return case, q, kc, vc, bt, cl


def _call_static(q, kc, vc, bt, cl, scale):
    from llm_from_scratch_b200 import _lib, ops
    B, Hq, D = q.shape
    nb, bs, Hkv, _ = kc.shape
    out = torch.full_like(q, float("nan"))
    rc = _lib.lib.b200_paged_decode_gqa_static(
        q.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(), bt.data_ptr(), bt.stride(0),
        cl.data_ptr(), B, Hq, Hkv, D, bs, nb, scale, _lib.DTYPE_BF16,
        ops.status_word(q.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
    return rc, out


def test_static_scratch_decode_matches_workspace_decode_twice_in_a_row():
    from llm_from_scratch_b200 import ops
    # long contexts so that sequences are cut across CTAs and the scratch is really used
    first = _case([5000, 33, 1, 2100, 0, 777], 32, 8, 128, seed=11)
    second = _case([300, 4097, 64], 32, 8, 128, seed=12)
    for case, q, kc, vc, bt, cl in (first, second):
        want = ops.paged_decode_gqa(q, kc, vc, bt, cl, 128 ** -0.5)
        rc, got = _call_static(q, kc, vc, bt, cl, 128 ** -0.5)
        assert rc == 0
        ops.check_status()
        assert torch.isfinite(got.float()).all()
        assert (got.float() - want.float()).abs().max().item() <= BF16_MAX_ABS


def test_static_scratch_decode_refuses_shapes_beyond_its_capacity():
    from llm_from_scratch_b200 import _lib
    # 128 query heads x head_dim 128: the partial-result scratch alone is ~19 MB > 8 MiB
    case, q, kc, vc, bt, cl = _case([40, 40], 128, 8, 128, seed=13)
    need = _lib.lib.b200_paged_decode_gqa_workspace_bytes(2, 128, 8, 128, _lib.DTYPE_BF16)
    assert need > (8 << 20)
    rc, out = _call_static(q, kc, vc, bt, cl, 128 ** -0.5)
    assert rc == ERR_TOO_LARGE
    assert b"scratch" in _lib.lib.b200_strerror(rc)
    assert torch.isnan(out.float()).all()  # nothing was launched
