"""Generation on the GPU: CUDA-graph decode against the eager KV-cache decode, native attention forward on the prefill."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _model():
    from sample_efficient_gpt_b200.config_schema import ModelConfig
    from sample_efficient_gpt_b200.models import build_model

    torch.manual_seed(0)
    cfg = ModelConfig(d_model=256, d_ff=512, n_layers=3, n_heads=4, n_kv_heads=2, vocab_size=512, attn_qknorm=True, attn_val_residual=True,
                      attn_gating="per-head", layernorm_scaling=True, weight_tying=False)
    return build_model(cfg).cuda().eval()


class _Tok:
    eos_token_id = None
    chat_template = None

    def get_vocab(self):
        return {}

    def decode(self, ids, skip_special_tokens=True):
        return " ".join(map(str, ids))


def test_graph_decode_matches_eager_decode():
    from sample_efficient_gpt_b200.evals.generation import ChatEngine, SamplingParams

    model = _model()
    eager = ChatEngine(model, _Tok(), "cuda", max_model_len=96, dtype=torch.float32, cuda_graphs=False)
    graph = ChatEngine(model, _Tok(), "cuda", max_model_len=96, dtype=torch.float32, cuda_graphs=True)
    assert not graph.fused_decode  # fp32: the module-path graph decoder
    prompts = [[3, 4, 5, 6, 7], [9, 8, 7, 6, 5], [1, 2, 3]]
    p = SamplingParams(max_tokens=24, temperature=0.0)
    a = eager.generate_ids([list(x) for x in prompts], p)
    b = graph.generate_ids([list(x) for x in prompts], p)
    assert a == b and all(len(r[0]) == 24 for r in a)
    c = graph.generate_ids([[5, 5, 5, 5, 5], [2, 3, 4, 5, 6]], p)  # second use of the captured graph and its caches
    d = eager.generate_ids([[5, 5, 5, 5, 5], [2, 3, 4, 5, 6]], p)
    assert c == d
    assert graph._decoders and all(dec.graph is not None for dec in graph._decoders.values())
    s = graph.generate_ids([[3, 4, 5]], SamplingParams(n=4, max_tokens=8, temperature=1.0, top_k=20, seed=3))
    assert len(s[0]) == 4 and all(len(x) == 8 for x in s[0])


def test_fused_engine_decode_tracks_module_decode():
    """bf16 decode on the engine's fused kernels (CUDA graph) against the bf16 module path: same greedy tokens while the
    top-2 logit gap is not within bf16 noise, and close logits at every compared step."""
    from sample_efficient_gpt_b200.evals.generation import ChatEngine, EngineDecoder, GraphDecoder, SamplingParams

    model = _model()
    fused = ChatEngine(model, _Tok(), "cuda", max_model_len=128, cuda_graphs=True)
    assert fused.fused_decode
    out = fused.generate_ids([[3, 4, 5, 6, 7, 8, 9, 10]], SamplingParams(max_tokens=16, temperature=0.0))
    assert len(out[0][0]) == 16 and isinstance(fused._decoders[1], EngineDecoder) and fused._decoders[1].graph is not None
    # step-by-step logits of both decoders on the same token stream
    a = EngineDecoder(model, 2, 64, "cuda")
    b = GraphDecoder(model, 2, 64, "cuda", torch.autocast("cuda", dtype=torch.bfloat16))
    prompt = torch.tensor([[3, 4, 5, 6, 7], [9, 8, 7, 6, 5]], device="cuda")
    la, lb = a.prefill(prompt), b.prefill(prompt)
    for _ in range(6):
        assert torch.allclose(la.float(), lb.float(), atol=0.15, rtol=0.05), float((la.float() - lb.float()).abs().max())
        nxt = lb.float().argmax(-1)
        la, lb = a.step(nxt), b.step(nxt)
