"""Config-5-shaped end-to-end check: a random-init Qwen3-architecture model whose decoder linears all
run through the new kernels, against the same model in the reference's `dequant_matmul` mode."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _build(layers):
    from transformers import Qwen3Config, Qwen3ForCausalLM
    from llmrqt_sdv1_b200.hf_adapter import quantize_model_
    cfg = Qwen3Config(hidden_size=2048, num_hidden_layers=layers, num_attention_heads=16, num_key_value_heads=8,
                      head_dim=128, intermediate_size=6144, vocab_size=151936, max_position_embeddings=4096,
                      tie_word_embeddings=False)
    torch.manual_seed(0)
    with torch.device("cuda"):
        model = Qwen3ForCausalLM(cfg).half().eval()
    n = quantize_model_(model, 128)
    assert n == 7 * layers
    return model


@torch.no_grad()
def test_qwen3_shaped_model_prefill_and_decode_parity():
    from llmrqt_sdv1_b200 import kernels
    from llmrqt_sdv1_b200.hf_adapter import set_impl_mode
    torch.backends.cuda.enable_cudnn_sdp(False)   # its per-shape plan building dominates a short test
    model = _build(layers=4)                       # 4 of the 28 layers keep the test short; shapes are config 5's
    g = torch.Generator(device="cuda").manual_seed(0)
    prompt = torch.randint(0, 151936, (1, 128), device="cuda", generator=g)

    set_impl_mode(model, "auto")
    out = model.generate(prompt, max_new_tokens=16, do_sample=False, use_cache=True)
    assert out.shape == (1, 144)
    logits_new = model(out).logits.float()         # prefill of the whole sequence: GEMM path (M = 144)
    step = model(out[:, :128], use_cache=True)
    dec_new = model(out[:, 128:129], past_key_values=step.past_key_values, use_cache=True).logits.float()  # GEMV, M = 1

    set_impl_mode(model, "dequant_matmul")
    logits_ref = model(out).logits.float()
    step = model(out[:, :128], use_cache=True)
    dec_ref = model(out[:, 128:129], past_key_values=step.past_key_values, use_cache=True).logits.float()
    torch.cuda.synchronize()
    assert kernels.gemm_status() == 0 and kernels.gemv_status() == 0

    # 4 layers x 7 linears compound the per-layer 2e-3 bound; 1e-2 of max|logit| holds with margin
    err_prefill = float((logits_new - logits_ref).abs().max() / logits_ref.abs().max())
    err_decode = float((dec_new - dec_ref).abs().max() / dec_ref.abs().max())
    assert err_prefill <= 1e-2, err_prefill
    assert err_decode <= 1e-2, err_decode
    # teacher-forced greedy choices agree wherever the reference's own top-2 margin exceeds the error
    top2 = logits_ref[0, 127:-1].topk(2, dim=-1).values
    confident = (top2[:, 0] - top2[:, 1]) > 2 * err_prefill * logits_ref.abs().max()
    agree = logits_new[0, 127:-1].argmax(-1) == logits_ref[0, 127:-1].argmax(-1)
    assert bool(agree[confident].all())


@torch.no_grad()
def test_fused_mlp_in_model():
    """`fuse_mlp_` swaps every layer's MLP for the two-launch form; prefill and decode logits stay within
    the compounded layer bound of the unfused model's."""
    from llmrqt_sdv1_b200 import AWQGatedMLP, kernels
    from llmrqt_sdv1_b200.hf_adapter import fuse_mlp_, set_impl_mode
    torch.backends.cuda.enable_cudnn_sdp(False)
    model = _build(layers=2)
    set_impl_mode(model, "auto")
    g = torch.Generator(device="cuda").manual_seed(1)
    ids = torch.randint(0, 151936, (1, 96), device="cuda", generator=g)
    ref_prefill = model(ids).logits.float()
    step = model(ids[:, :95], use_cache=True)
    ref_decode = model(ids[:, 95:96], past_key_values=step.past_key_values, use_cache=True).logits.float()
    assert fuse_mlp_(model) == 2
    assert all(isinstance(layer.mlp, AWQGatedMLP) for layer in model.model.layers)
    new_prefill = model(ids).logits.float()
    step = model(ids[:, :95], use_cache=True)
    new_decode = model(ids[:, 95:96], past_key_values=step.past_key_values, use_cache=True).logits.float()
    torch.cuda.synchronize()
    assert kernels.gemm_status() == 0 and kernels.gemv_status() == 0
    assert float((new_prefill - ref_prefill).abs().max() / ref_prefill.abs().max()) <= 1e-2
    assert float((new_decode - ref_decode).abs().max() / ref_decode.abs().max()) <= 1e-2


@torch.no_grad()
def test_fused_qkv_attention_in_model():
    """`fuse_qkv_` replaces q/k/v by one linear of 4096 columns (the shape the reference's fuser builds):
    same logits as the three separate linears up to the kernels' summation order."""
    from llmrqt_sdv1_b200 import kernels
    from llmrqt_sdv1_b200.hf_adapter import FusedQKVAttention, fuse_qkv_, set_impl_mode
    torch.backends.cuda.enable_cudnn_sdp(False)
    model = _build(layers=2)
    set_impl_mode(model, "auto")
    g = torch.Generator(device="cuda").manual_seed(2)
    ids = torch.randint(0, 151936, (1, 64), device="cuda", generator=g)
    ref_prefill = model(ids).logits.float()
    step = model(ids[:, :63], use_cache=True)
    ref_decode = model(ids[:, 63:64], past_key_values=step.past_key_values, use_cache=True).logits.float()
    assert fuse_qkv_(model) == 2
    attn = model.model.layers[0].self_attn
    assert isinstance(attn, FusedQKVAttention) and attn.qkv_proj.out_features == 4096
    new_prefill = model(ids).logits.float()
    step = model(ids[:, :63], use_cache=True)
    new_decode = model(ids[:, 63:64], past_key_values=step.past_key_values, use_cache=True).logits.float()
    torch.cuda.synchronize()
    assert kernels.gemm_status() == 0 and kernels.gemv_status() == 0
    assert float((new_prefill - ref_prefill).abs().max() / ref_prefill.abs().max()) <= 1e-2
    assert float((new_decode - ref_decode).abs().max() / ref_decode.abs().max()) <= 1e-2


@torch.no_grad()
def test_graphed_decoder_all_28_layers():
    """Config 5 in full depth: the whole decode step captured in one CUDA graph gives the tokens of the same
    step run eagerly, its logits stay within the compounded layer bound of the `dequant_matmul` model's, and
    its greedy tokens agree with Hugging Face's `generate` wherever the reference's top-2 margin is clear."""
    from llmrqt_sdv1_b200 import kernels
    from llmrqt_sdv1_b200.decoder import GraphedDecoder
    from llmrqt_sdv1_b200.hf_adapter import fuse_mlp_, fuse_qkv_, set_impl_mode
    torch.backends.cuda.enable_cudnn_sdp(False)
    model = _build(layers=28)
    g = torch.Generator(device="cuda").manual_seed(0)
    prompt = torch.randint(0, 151936, (1, 128), device="cuda", generator=g)
    set_impl_mode(model, "dequant_matmul")
    seq_ref = model.generate(prompt, max_new_tokens=24, min_new_tokens=24, do_sample=False)
    logits_ref = model(seq_ref).logits.float()
    set_impl_mode(model, "auto")
    assert fuse_qkv_(model) == 28 and fuse_mlp_(model) == 28

    eager = GraphedDecoder(model, max_len=192, capture=False)
    seq_eager = eager.generate(prompt, 24)
    graphed = GraphedDecoder(model, max_len=192)
    seq_graph = graphed.generate(prompt, 24)
    seq_again = graphed.generate(prompt, 24)
    torch.cuda.synchronize()
    assert graphed.graph is not None
    assert torch.equal(seq_graph, seq_eager), "graph replay and eager steps disagree"
    assert torch.equal(seq_graph, seq_again), "two generations from the same prompt disagree"
    assert kernels.gemm_status() == 0 and kernels.gemv_status() == 0

    # 28 layers x 4 fused linears compound the per-layer 2e-3 bound
    err = graphed.teacher_forced_error(seq_ref, logits_ref)
    assert err <= 2e-2, err
    # greedy tokens: equal to the reference's wherever its own top-2 margin exceeds twice the logit error,
    # up to the first position where the sequences part (after that the inputs differ)
    ref_new, got_new = seq_ref[0, 128:].tolist(), seq_graph[0, 128:].tolist()
    top2 = logits_ref[0, 127:-1].topk(2, dim=-1).values
    margin = (top2[:, 0] - top2[:, 1]) / logits_ref.abs().max()
    for i, (a, b) in enumerate(zip(ref_new, got_new)):
        if a != b:
            assert float(margin[i]) <= 2 * err, f"token {i} differs although the reference margin is clear"
            break

    # a long context: the attention launch with the cached positions cut into chunks (one CTA per head and chunk)
    # against one CTA per head - the first decode step after the same 700-token prefill
    long_prompt = torch.randint(0, 151936, (1, 700), device="cuda", generator=g)
    chunks = GraphedDecoder(model, max_len=1024)
    one_cta = GraphedDecoder(model, max_len=1024, attn_split=False)
    assert chunks._attn_split and not one_cta._attn_split and not graphed._attn_split
    s1, s2 = chunks.generate(long_prompt, 2), one_cta.generate(long_prompt, 2)
    torch.cuda.synchronize()
    l1, l2 = chunks._graph_logits.float(), one_cta._graph_logits.float()
    assert torch.equal(s1[:, :701], s2[:, :701])
    assert float((l1 - l2).abs().max() / l2.abs().max()) <= 1e-2      # last-bit differences of 28 attention outputs, compounded
    assert chunks.time_step_at(900, iters=3) > 0.0
    assert torch.equal(chunks.generate(long_prompt, 2), s1)           # the timing hook restored the state
    assert kernels.gemm_status() == 0 and kernels.gemv_status() == 0
