"""Host-side check of the per-token decode step that `GraphedDecoder` captures: on CPU (no graph, plain
nn.Linear projections) its prefill logits, its cached single-token steps and its greedy tokens must match
Hugging Face's own forward / generate on a tiny random Qwen3-architecture model."""
import pytest
import torch


def _tiny(seed=0):
    from transformers import Qwen3Config, Qwen3ForCausalLM
    cfg = Qwen3Config(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                      intermediate_size=128, vocab_size=97, max_position_embeddings=64, tie_word_embeddings=False)
    torch.manual_seed(seed)
    return Qwen3ForCausalLM(cfg).float().eval()


@torch.no_grad()
def test_decoder_matches_hf_forward_and_generate():
    from llmrqt_sdv1_b200.decoder import GraphedDecoder
    model = _tiny()
    ids = torch.randint(0, 97, (1, 12), generator=torch.Generator().manual_seed(1))
    dec = GraphedDecoder(model, max_len=40)
    ref = model(ids).logits
    mine = dec.forward_tokens(ids)
    assert float((mine - ref).abs().max()) <= 1e-4 * float(ref.abs().max())
    # cached decoding: greedy tokens equal to Hugging Face's, and each step's logits equal to a full forward
    want = model.generate(ids, max_new_tokens=10, min_new_tokens=10, do_sample=False)
    got = dec.generate(ids, 10)
    assert torch.equal(got, want)
    dec.prefill(ids)
    step_logits = dec.step_eager()                       # consumes the first generated token
    full = model(want[:, :13]).logits[:, -1:]
    assert float((step_logits - full).abs().max()) <= 1e-4 * float(full.abs().max())
    assert dec.teacher_forced_error(want, model(want).logits) <= 1e-4


def test_decoder_rejects_overlong_requests():
    from llmrqt_sdv1_b200.decoder import GraphedDecoder
    dec = GraphedDecoder(_tiny(), max_len=16)
    with pytest.raises(ValueError):
        dec.generate(torch.zeros((1, 10), dtype=torch.long), 8)
    with pytest.raises(ValueError):
        dec.forward_tokens(torch.zeros((1, 17), dtype=torch.long))
