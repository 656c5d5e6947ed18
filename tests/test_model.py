import pytest
import torch

from sample_efficient_gpt_b200.models import KVCache, Transformer

KW = dict(attn_qknorm=True, attn_val_residual=True, attn_gating="per-head", layernorm_scaling=True, n_kv_heads=2, weight_tying=True)

EXPECTED_KEYS_BLOCK0 = [
    "blocks.0.ln1.gain", "blocks.0.attn.alpha1", "blocks.0.attn.alpha2", "blocks.0.attn.scale",
    "blocks.0.attn.qkv.linear.weight", "blocks.0.attn.out.linear.weight", "blocks.0.attn.sdpa_qknorm.gain",
    "blocks.0.attn.attn_gate.linear.weight", "blocks.0.ln2.gain", "blocks.0.ffn.up.linear.weight",
    "blocks.0.ffn.down.linear.weight",
]


def _perturb(m):
    with torch.no_grad():
        for b in m.blocks:
            b.attn.alpha1.fill_(0.8); b.attn.alpha2.fill_(0.5); b.attn.scale.fill_(1.1); b.attn.sdpa_qknorm.gain.fill_(1.3)
            b.ln1.gain.add_(torch.randn_like(b.ln1.gain) * 0.1)


def test_state_dict_layout():
    m = Transformer(2, 100, 128, 4, 200, **KW)
    keys = list(m.state_dict().keys())
    assert keys[0] == "embedding.weight"
    assert keys[1:12] == EXPECTED_KEYS_BLOCK0
    assert keys[-3:] == ["final_norm.gain", "lm_head.weight", "lm_head.linear.weight"]
    sd = m.state_dict()
    assert sd["lm_head.weight"].data_ptr() == sd["embedding.weight"].data_ptr()  # stored alias of the embedding
    assert sd["lm_head.linear.weight"].data_ptr() != sd["embedding.weight"].data_ptr()  # the real head is untied
    assert "lm_head.weight" not in dict(m.named_parameters())
    assert m.blocks[0].ffn.up.linear.weight.shape == (2 * 192, 128)  # d_ff floored to a multiple of 64
    assert float(m.blocks[1].ln1.position_scale) == pytest.approx(2**-0.5) and float(m.final_norm.position_scale) == 1.0
    assert all(v.dtype == torch.float32 for v in sd.values())
    m2 = Transformer(2, 100, 128, 4, 200, n_kv_heads=2)
    assert "blocks.0.attn.alpha1" not in m2.state_dict() and "lm_head.weight" not in m2.state_dict()


def test_matches_reference_model(reference_path):
    from sample_efficient_gpt.transformer import Transformer as RefT

    torch.manual_seed(0)
    ref = RefT(3, 1000, 128, 4, 256, **KW)
    torch.manual_seed(0)
    mine = Transformer(3, 1000, 128, 4, 256, **KW)
    assert list(ref.state_dict().keys()) == list(mine.state_dict().keys())
    assert [n for n, _ in ref.named_parameters()] == [n for n, _ in mine.named_parameters()]
    assert all(torch.equal(a, b) for a, b in zip(ref.state_dict().values(), mine.state_dict().values()))  # same seed, same init
    _perturb(ref)
    mine.load_state_dict(ref.state_dict())
    ids = torch.randint(0, 1000, (2, 17))
    lr, kr = ref(ids)
    lm, km = mine(ids)
    assert torch.allclose(lr, lm, atol=2e-5) and torch.allclose(kr, km, atol=1e-5)
    lr.square().mean().backward()
    lm.square().mean().backward()
    for (n, a), b in zip(ref.named_parameters(), mine.parameters()):
        assert torch.allclose(a.grad, b.grad, atol=1e-6), n
    g1, _ = ref.generate(ids[:1, :5], 0, temperature=0.0, max_steps=6)
    g2, _ = mine.generate(ids[:1, :5], 0, temperature=0.0, max_steps=6)
    assert torch.equal(g1, g2)


@pytest.mark.parametrize("gating", [False, "elementwise", "per-head", "per-head-hd"])
def test_kv_cache_decoding_matches_full_forward(gating):
    torch.manual_seed(1)
    m = Transformer(2, 50, 64, 4, 128, attn_qknorm=True, attn_val_residual=True, attn_gating=gating, layernorm_scaling=True, n_kv_heads=2)
    _perturb(m)
    m.eval()
    ids = torch.randint(0, 50, (2, 9))
    full, _ = m(ids)
    caches = [KVCache() for _ in range(2)]
    a, _ = m(ids[:, :6], kv_cache=caches)
    outs = [a]
    for t in range(6, 9):
        o, _ = m(ids[:, t : t + 1], kv_cache=caches)
        outs.append(o)
    assert torch.allclose(torch.cat(outs, 1), full, atol=1e-4)


def test_generate_sampling_and_checkpointing():
    torch.manual_seed(2)
    m = Transformer(2, 50, 64, 4, 128, num_grad_checkpoint_layers=1, **KW)
    out, eos = m.generate(torch.randint(0, 50, (1, 4)), eos_token_id=0, top_p=0.5, temperature=0.8, max_steps=5)
    assert out.shape[1] <= 9 and eos is not None
    ids = torch.randint(0, 50, (2, 8))
    m.train()
    l1, _ = m(ids)
    m.num_grad_checkpoint_layers = 0
    l2, _ = m(ids)
    assert torch.allclose(l1, l2, atol=1e-6)
    l1.sum().backward()


def test_mup_base_width_scales_logits():
    torch.manual_seed(3)
    a = Transformer(1, 30, 128, 2, 128, mup_base_width=64)
    assert a.output_mult == 0.5
    ids = torch.randint(0, 30, (1, 4))
    h, _ = a.hidden_states(ids)
    assert torch.allclose(a(ids)[0], a.lm_head(h) * 0.5)
