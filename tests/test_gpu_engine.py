"""The fused engine on a GPU in bf16 against the fp32 module path, and the smoke entry point."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _model(ckpt=0):
    from sample_efficient_gpt_b200.models import Transformer

    torch.manual_seed(0)
    m = Transformer(3, 4096, 256, 4, 768, attn_qknorm=True, attn_val_residual=True, attn_gating="per-head",
                    layernorm_scaling=True, n_kv_heads=2, weight_tying=True, num_grad_checkpoint_layers=ckpt)
    with torch.no_grad():
        for b in m.blocks:
            b.attn.alpha1.fill_(0.9); b.attn.alpha2.fill_(0.4); b.attn.scale.fill_(1.05); b.attn.sdpa_qknorm.gain.fill_(1.2)
    return m


@pytest.mark.parametrize("ckpt", [0, 2])
def test_engine_bf16_close_to_fp32_autograd(ckpt):
    from sample_efficient_gpt_b200 import ops
    from sample_efficient_gpt_b200.training.engine import FusedEngine
    from sample_efficient_gpt_b200.training.loss import efficient_cross_entropy

    m = _model(ckpt).cuda()
    ids = torch.randint(0, 4096, (2, 256), device="cuda")
    tg = torch.randint(0, 4096, (2, 256), device="cuda")
    logits, kurt = m(ids)
    loss, _, _ = efficient_cross_entropy(logits, tg)
    loss.backward()
    ref = {n: p.grad.clone() for n, p in m.named_parameters()}
    for p in m.parameters():
        p.grad = None
    before = ops.launch_count
    eng = FusedEngine(m, torch.bfloat16)
    out = eng.forward_backward(ids, tg, 1.0)
    assert ops.launch_count > before
    assert abs(float(out.loss) - float(loss)) < 0.05
    assert torch.allclose(out.kurtosis, kurt.float(), rtol=0.05, atol=0.05)
    for n, p in m.named_parameters():
        g, r = p.grad.float(), ref[n].float()
        if g.numel() == 1:  # scalar gradients are sums of many bf16-rounded terms of both signs: absolute slack
            assert (g - r).abs().item() < 0.1 * r.abs().item() + 5e-3, f"{n}: {g.item()} vs {r.item()}"
            continue
        cos = torch.nn.functional.cosine_similarity(g.flatten(), r.flatten(), dim=0)
        assert cos > 0.98, f"{n}: cosine {cos}"
        assert (g.norm() / (r.norm() + 1e-12) - 1).abs() < 0.1, n
    ev = eng.forward_loss(ids, tg)
    assert abs(float(ev.loss) - float(loss)) < 0.05


def test_smoke_entry_point():
    import __graft_entry__ as g

    g.smoke()


def test_trainer_loss_goes_down_on_gpu(tmp_path):
    import numpy as np

    from sample_efficient_gpt_b200.training.trainer import Trainer
    from sample_efficient_gpt_b200.utils.config_tools import apply_overrides, load_cfg

    rng = np.random.default_rng(0)
    d = tmp_path / "train"; d.mkdir()
    np.save(d / "a.npy", rng.integers(0, 512, 200_000).astype(np.uint16))
    np.save(tmp_path / "val.npy", rng.integers(0, 512, 20_000).astype(np.uint16))
    cfg = load_cfg("tiny_cpu.yaml")
    cfg = apply_overrides(cfg, {"trainer.device": "cuda", "trainer.dtype": "bfloat16", "data.train_path": str(d),
                                "data.validation_path": str(tmp_path / "val.npy"), "trainer.save_dir": str(tmp_path / "ck"),
                                "trainer.max_steps": 12, "trainer.ema_every": 2, "model.vocab_size": 4096})
    tr = Trainer(cfg)
    losses = []
    for _ in range(12):
        x, y = tr.fetch_batch()
        losses.append(float(tr.train_step(x, y)["train_loss"]))
        tr.iteration += 1
    assert losses[-1] < losses[0] - 0.5, losses
    v = tr.validate()
    assert v["val_loss"] == v["val_loss"]
    tr.save_state()
    assert (tmp_path / "ck" / "12.pt").exists() and (tmp_path / "ck" / "12_ema.pt").exists()
