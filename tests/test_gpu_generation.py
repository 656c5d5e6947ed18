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
