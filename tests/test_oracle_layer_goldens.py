"""The CPU oracle under autocast against the reference's own modules at the benchmark layer shapes
(fixtures of tests/golden/make_golden_layers.py): the MoE layer of the GQA+MoE decoder (d_model 1024,
16 experts top-2 + shared, d_ff 704) and the latent attention of the MLA+MoE decoder (16 heads,
kv_lora_rank 512, q_lora_rank 1024, rope_dim 64).  Same torch operators in the same order, so the
oracle reproduces the bf16 outputs bit for bit (MoE layer, latent rows, decode steps) or to one rounding
step on a few elements (the 300-token latent-attention prefill)."""
import numpy as np
import torch

from oracle.model import OracleModel

from layer_fixtures import MLA_LAYER, MOE_LAYER, checked_input, from_bf16_bits, layer_weights, load


def test_moe_layer_of_the_gqa_moe_decoder_bf16_autocast():
    z = load("moe_layer_c3.npz")
    m = OracleModel(MOE_LAYER, layer_weights(MOE_LAYER, z, "layers.0.ffn."))
    rows = int(z["decode_rows"])
    x = checked_input(z, "decode_input_seed", "decode_input_sum", rows, 1024)
    with torch.no_grad(), torch.autocast("cpu", dtype=torch.bfloat16):
        y = m._moe(x, "layers.0.ffn")
    want = from_bf16_bits(z["decode_out"])
    assert y.dtype == torch.bfloat16 and torch.equal(y[torch.from_numpy(z["decode_kept"])], want)


def test_latent_attention_of_the_mla_moe_decoder_bf16_autocast():
    z = load("mla_layer_c4.npz")
    m = OracleModel(MLA_LAYER, layer_weights(MLA_LAYER, z, "layers.0.att."))
    P, Dn = int(z["prefill"]), int(z["decode"])
    x = checked_input(z, "input_seed", "input_sum", P + Dn, 2048)
    cache = m.new_cache(512)[0]
    outs = []
    with torch.no_grad(), torch.autocast("cpu", dtype=torch.bfloat16):
        outs.append(m._mla(x[:P], "layers.0.att", 0, torch.tril(torch.ones(P, P, dtype=torch.bool)), cache))
        for i in range(Dn):
            outs.append(m._mla(x[P + i:P + i + 1], "layers.0.att", P + i, None, cache))
    y = torch.cat(outs)
    want = from_bf16_bits(z["out"])
    assert y.dtype == torch.bfloat16
    # the cached latent rows (what the paged pool must hold) and the outputs
    np.testing.assert_array_equal(cache["kv"][:P + Dn].to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16),
                                  z["latent"])
    # decode rows bit for bit; prefill rows to one bf16 rounding step on a fraction of a percent of the elements
    # (the CPU bf16 einsum kernels choose their blocking from operand strides, which the restatement does not copy)
    assert torch.equal(y[P:], want[P:])
    diff = (y[:P].float() - want[:P].float()).abs()
    assert diff.max().item() <= 2.0 ** -10 and (diff > 0).float().mean().item() < 0.01
