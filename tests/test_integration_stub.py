"""Executes the reference-side binding printed in INTEGRATION.md: the ``Attention`` layer a maintainer of the
reference would add (ctypes + torch only) and the ``compute_hash`` replacement.  The code blocks are taken
from the document as they stand; only the library path placeholder is filled in and the reference's
``utils.context`` module is stood in for by this package's identical one."""
import os
import re
import sys
import types

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _code_blocks():
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    return re.findall(r"```python\n(.*?)```", text, flags=re.S)


def _load_stub():
    from llm_from_scratch_b200 import _lib
    from llm_from_scratch_b200.utils import context
    attention_src, hash_src = _code_blocks()[:2]
    assert "class Attention" in attention_src and "def compute_hash" in hash_src
    attention_src = re.sub(r'B200_LIBRARY_PATH = ".*?"', f'B200_LIBRARY_PATH = "{_lib.LIB_PATH}"', attention_src)
    utils_pkg = types.ModuleType("utils")
    utils_pkg.context = context
    saved = {k: sys.modules.get(k) for k in ("utils", "utils.context")}
    sys.modules["utils"], sys.modules["utils.context"] = utils_pkg, context
    try:
        ns = {}
        exec(compile(attention_src, "INTEGRATION.md:attention", "exec"), ns)
        exec(compile(hash_src, "INTEGRATION.md:compute_hash", "exec"), ns)
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
    return ns


def test_compute_hash_binding_gives_the_reference_hashes():
    """Known answers produced by the reference's BlockManager.compute_hash (xxhash of the int32 token ids,
    chained through the previous block's hash)."""
    ns = _load_stub()
    h0 = ns["compute_hash"](None, list(range(16)), -1)
    assert h0 == 9963129416833264760
    assert ns["compute_hash"](None, list(range(16, 32)), h0) == 2400706462553290651
    assert ns["compute_hash"](None, [0] * 16, -1) == 2700762989836380697


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_attention_binding_prefill_then_decode_against_the_oracle(dtype):
    """One ragged prefill step (the call also scatters K/V into the paged pool), one prefill step over a cached
    prefix (block tables), and one decode step, driven through the global Context exactly as the reference's
    model runner would, against the CPU oracle."""
    from llm_from_scratch_b200.utils.context import reset_context, set_context
    from oracle import attention as orc
    ns = _load_stub()
    Hq, Hkv, D, bs, nblk = 8, 2, 64, 16, 40
    tol = 2e-2 if dtype == torch.bfloat16 else 2e-5
    layer = ns["Attention"](Hq, D, D ** -0.5, Hkv)
    kc = torch.zeros(nblk, bs, Hkv, D, dtype=dtype, device="cuda")
    vc = torch.zeros_like(kc)
    layer.k_cache, layer.v_cache = kc, vc
    g = torch.Generator().manual_seed(3)
    lens = [37, 5, 64]
    T = sum(lens)
    q, k, v = (torch.randn(T, h, D, generator=g).to(dtype) for h in (Hq, Hkv, Hkv))
    perm = np.random.default_rng(0).permutation(nblk).astype(np.int32)
    tables, pos = [], 0
    for n in lens:
        nb = (n + 1 + bs - 1) // bs                      # room for one decoded token
        tables.append(perm[pos:pos + nb])
        pos += nb
    slots = np.concatenate([tables[i][np.arange(n) // bs].astype(np.int64) * bs + np.arange(n) % bs
                            for i, n in enumerate(lens)])
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    # ---- prefill of new sequences
    set_context(True, cu.cuda(), cu.cuda(), max(lens), max(lens), torch.from_numpy(slots).cuda(), None, None)
    o = layer(q.cuda(), k.cuda(), v.cuda())
    torch.cuda.synchronize()
    want = orc.prefill_varlen(q, k, v, cu, cu, D ** -0.5)
    assert (o.float().cpu() - want).abs().max().item() <= tol
    kc_ref, vc_ref = torch.zeros(nblk, bs, Hkv, D, dtype=dtype), torch.zeros(nblk, bs, Hkv, D, dtype=dtype)
    orc.store_kvcache(k, v, kc_ref, vc_ref, torch.from_numpy(slots))
    assert torch.equal(kc.cpu(), kc_ref) and torch.equal(vc.cpu(), vc_ref)
    # ---- decode: one more token per sequence
    qd, kd, vd = (torch.randn(3, h, D, generator=g).to(dtype) for h in (Hq, Hkv, Hkv))
    dslots = np.array([tables[i][n // bs] * bs + n % bs for i, n in enumerate(lens)], dtype=np.int64)
    width = max(len(t) for t in tables)
    bt = np.full((3, width), -1, dtype=np.int32)
    for i, t in enumerate(tables):
        bt[i, :len(t)] = t
    clens = np.array([n + 1 for n in lens], dtype=np.int64)
    set_context(False, slot_mapping=torch.from_numpy(dslots).cuda(), context_lens=torch.from_numpy(clens).cuda(),
                block_tables=torch.from_numpy(bt).cuda())
    od = layer(qd.cuda(), kd.cuda(), vd.cuda())
    torch.cuda.synchronize()
    orc.store_kvcache(kd, vd, kc_ref, vc_ref, torch.from_numpy(dslots))
    wantd = orc.paged_decode_gqa(qd, kc_ref, vc_ref, bt, clens, D ** -0.5)
    assert (od.float().cpu() - wantd).abs().max().item() <= tol
    # ---- prefill of 9 more tokens of sequence 1 over its cached 6-token context (block tables set)
    n_old, n_new = lens[1] + 1, 9
    q2, k2, v2 = (torch.randn(n_new, h, D, generator=g).to(dtype) for h in (Hq, Hkv, Hkv))
    p = np.arange(n_old, n_old + n_new)
    slots2 = tables[1][p // bs].astype(np.int64) * bs + p % bs
    set_context(True, torch.tensor([0, n_new], dtype=torch.int32).cuda(),
                torch.tensor([0, n_old + n_new], dtype=torch.int32).cuda(), n_new, n_old + n_new,
                torch.from_numpy(slots2).cuda(), None, torch.from_numpy(bt[1:2].copy()).cuda())
    o2 = layer(q2.cuda(), k2.cuda(), v2.cuda())
    torch.cuda.synchronize()
    orc.store_kvcache(k2, v2, kc_ref, vc_ref, torch.from_numpy(slots2))
    rows = torch.from_numpy(np.concatenate([tables[1][np.arange(n_old + n_new) // bs].astype(np.int64) * bs
                                            + np.arange(n_old + n_new) % bs]))
    k_all, v_all = kc_ref.view(-1, Hkv, D)[rows], vc_ref.view(-1, Hkv, D)[rows]
    want2 = orc.prefill_varlen(q2, k_all, v_all, torch.tensor([0, n_new], dtype=torch.int32),
                               torch.tensor([0, n_old + n_new], dtype=torch.int32), D ** -0.5)
    assert (o2.float().cpu() - want2).abs().max().item() <= tol
    reset_context()
