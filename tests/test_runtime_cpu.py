"""Prefill of the decode runtime against a Hugging Face Llama of the same (tiny) shape, fp32 on CPU:
the caller-side plumbing around the attention path (weight layout, RoPE, chunking, cache layout
[B, T, KVH, D]) follows the model the reference runtime drives (tutorial_code/runtime_common.py:274-397)."""
import pytest
import torch

from santa_b200.runtime import DecodeRuntime, LlamaShape


@pytest.fixture(scope="module")
def tiny_hf():
    transformers = pytest.importorskip("transformers")
    cfg = transformers.LlamaConfig(hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=1, head_dim=128, vocab_size=1000,
                                   rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=4096,
                                   tie_word_embeddings=False, attention_bias=False, mlp_bias=False)
    torch.manual_seed(0)
    return transformers.LlamaForCausalLM(cfg).eval()


SHAPE = LlamaShape(hidden=512, layers=2, heads=4, kv_heads=1, head_dim=128, intermediate=1024, vocab=1000)


@pytest.mark.parametrize("chunk", [16, 512])
def test_chunked_prefill_matches_hf(tiny_hf, chunk):
    ids = torch.randint(0, 1000, (2, 37), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = tiny_hf(input_ids=ids, use_cache=True)
    rt = DecodeRuntime(SHAPE, 2, 64, "cpu", dtype=torch.float32, attention="sdpa")
    rt.load_hf_state_dict(tiny_hf.state_dict())
    last = rt.prefill(ids, chunk=chunk)
    assert (last - ref.logits[:, -1].float()).abs().max().item() < 1e-4
    for li in range(2):
        layer = ref.past_key_values.layers[li]
        assert (rt.k_cache[li][:, :37].permute(0, 2, 1, 3) - layer.keys).abs().max().item() < 1e-4
        assert (rt.v_cache[li][:, :37].permute(0, 2, 1, 3) - layer.values).abs().max().item() < 1e-4
        assert (rt.k_cache[li][:, 37:] == 0).all()
    assert rt.pos.tolist() == [37, 37]


def test_runtime_argument_errors():
    with pytest.raises(RuntimeError, match="D=128"):
        DecodeRuntime(LlamaShape(hidden=256, layers=1, heads=4, kv_heads=1, head_dim=64, intermediate=512, vocab=100),
                      1, 8, "cpu", dtype=torch.float32, attention="sdpa")
    with pytest.raises(ValueError, match="unknown attention backend"):
        DecodeRuntime(SHAPE, 1, 8, "cpu", dtype=torch.float32, attention="fa2")
    rt = DecodeRuntime(SHAPE, 1, 8, "cpu", dtype=torch.float32, attention="sdpa")
    with pytest.raises(ValueError, match="prefill_chunk_size"):
        rt.prefill(torch.zeros(1, 4, dtype=torch.long), chunk=0)
    with pytest.raises(RuntimeError, match="does not fit"):
        rt.prefill(torch.zeros(1, 9, dtype=torch.long))
