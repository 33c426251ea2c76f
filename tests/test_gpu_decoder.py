"""The decode-graph glue (shared quantization between sibling projections, paged int4 cache, CUDA-graph
replay of the decode step) against the oracle's CPU statement of the same stack, and against itself
(graph replay == eager launches, bit for bit)."""
import pytest
import torch

from oracle.decoder import DecoderRef
from conftest import rel_l2
from signrot_b200.functional.hadamard import get_hadK
from signrot_b200.transformers import kernel_utils as ku

pytestmark = pytest.mark.gpu
DEV = "cuda"


def small_model(experts=0, layers=2, seed=0):
    cfg = ku.DecoderConfig(hidden_size=512, intermediate_size=1536, num_hidden_layers=layers, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=128, vocab_size=512, num_local_experts=experts,
                           num_experts_per_tok=2)
    with torch.device(DEV):
        model = ku.KernelDecoderModel(cfg)
    return model.to(DEV).random_init_(seed), cfg


def oracle_state(model, cfg):
    layers = []
    for layer in model.layers:
        at, mlp = layer.self_attn, layer.mlp
        d = {}
        for tag, lin in (("q", at.q_proj), ("k", at.k_proj), ("v", at.v_proj), ("o", at.o_proj),
                         ("g", mlp.gate_proj), ("u", mlp.up_proj), ("d", mlp.down_proj)):
            d["w" + tag] = lin.kernel_module.weight.cpu()
            d["s" + tag] = lin.kernel_module.weight_scales.cpu()
        d["sign_d"] = mlp.down_proj.kernel_hadamard.had_adj_sign.cpu()
        layers.append(d)
    hadK, K = get_hadK(cfg.intermediate_size)
    c = dict(hidden=cfg.hidden_size, heads=cfg.num_attention_heads, kv_heads=cfg.num_key_value_heads,
             head_dim=cfg.head_dim, ffn=cfg.intermediate_size, eps=cfg.rms_norm_eps, theta=cfg.rope_theta,
             hadK=hadK.to(torch.float16) if hadK is not None else None, K=K)
    return {"embed": model.embed_tokens.weight.detach().cpu(), "lm_head": model.lm_head.weight.detach().cpu(),
            "layers": layers}, c


@torch.no_grad()
def test_prefill_and_decode_match_oracle():
    model, cfg = small_model()
    B, T, steps, page = 2, 40, 3, 16
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab_size, (B, T), generator=g)
    nxt = [torch.randint(0, cfg.vocab_size, (B, 1), generator=g) for _ in range(steps)]
    state, c = oracle_state(model, cfg)
    ref = DecoderRef(state, c, B, page, T + steps)
    cache = ku.build_paged_cache(model, B, T + steps, page_size=page)

    want = ref.forward(prompt)
    got = model(prompt.to(DEV), past_key_values=cache).logits.cpu()
    assert torch.isfinite(got).all()
    # every one-ulp difference ahead of a quantizer can flip codes after it, so the bound for a
    # whole stack is the quantization-noise floor, not the single-operator 1e-3
    assert rel_l2(got, want) <= 2e-2
    for tok in nxt:
        want = ref.forward(tok)
        got = model(tok.to(DEV), past_key_values=cache).logits.cpu()
        assert got.shape == (B, 1, cfg.vocab_size)
        # decode adds the int4 cache on both sides; a glue error (position, page slot, head
        # mapping) shows as a relative error near 1, flipped rounding ties as a few 1e-2
        assert rel_l2(got, want) <= 5e-2
    assert cache.get_seq_length() == T + steps == ref.length


@torch.no_grad()
@pytest.mark.parametrize("experts", [0, 4])
def test_graph_replay_equals_eager(experts):
    model, cfg = small_model(experts=experts)
    B, T, page = 2, 30, 16
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, cfg.vocab_size, (B, T), generator=g).to(DEV)
    toks = [torch.randint(0, cfg.vocab_size, (B, 1), generator=g).to(DEV) for _ in range(4)]

    eager_cache = ku.build_paged_cache(model, B, T + 8, page_size=page)
    model(prompt, past_key_values=eager_cache)
    eager = [model(t, past_key_values=eager_cache).logits.clone() for t in toks]

    cache = ku.build_paged_cache(model, B, T + 8, page_size=page)
    model(prompt, past_key_values=cache)
    dec = ku.try_graph_decoder(model, cache, B)
    assert dec is not None, "the decode step must be capture-safe"
    assert cache.get_seq_length() == T            # capture and validation rewind the length
    for t, want in zip(toks, eager):
        got = dec.step(t)
        assert torch.equal(got, want)             # same kernels, same inputs: identical bits
    assert cache.get_seq_length() == T + len(toks)   # crosses a page boundary (30 -> 34, page 16)


@torch.no_grad()
def test_generate_graph_and_eager_agree():
    model, cfg = small_model(layers=1, seed=3)
    prompt = torch.randint(0, cfg.vocab_size, (2, 17), generator=torch.Generator().manual_seed(3)).to(DEV)
    a = ku.generate(model, prompt, 6, page_size=16, use_graph=True)
    b = ku.generate(model, prompt, 6, page_size=16, use_graph=False)
    assert a.shape == (2, 6) and torch.equal(a, b)


@torch.no_grad()
@pytest.mark.parametrize("experts", [0, 4])
def test_fused_edges_give_the_bits_of_the_separate_launches(experts):
    """add+RMSNorm+quantizer, one q/k/v GEMM, rope+append, gate/up+SwiGLU: every fused launch keeps
    the rounding points of the launches it replaces, so logits agree bit for bit."""
    cfg_kw = dict(hidden_size=512, intermediate_size=1536, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, head_dim=128, vocab_size=512, num_local_experts=experts)
    models = []
    for fuse in (True, False):
        with torch.device(DEV):
            m = ku.KernelDecoderModel(ku.DecoderConfig(fuse_edges=fuse, **cfg_kw))
        models.append(m.to(DEV).random_init_(5))
    fused, plain = models
    assert hasattr(fused.layers[0].self_attn, "qkv_fused") and not hasattr(plain.layers[0].self_attn, "qkv_fused")
    g = torch.Generator().manual_seed(9)
    prompt = torch.randint(0, 512, (2, 21), generator=g).to(DEV)
    toks = [torch.randint(0, 512, (2, 1), generator=g).to(DEV) for _ in range(3)]
    ca, cb = (ku.build_paged_cache(m, 2, 32, page_size=16) for m in models)
    assert torch.equal(fused(prompt, past_key_values=ca).logits, plain(prompt, past_key_values=cb).logits)
    for t in toks:
        assert torch.equal(fused(t, past_key_values=ca).logits, plain(t, past_key_values=cb).logits)


@torch.no_grad()
def test_checkpoint_reload_gives_the_same_logits(tmp_path):
    from signrot_b200 import checkpoint as ck
    model, cfg = small_model(seed=11)
    ck.save_packed_checkpoint(model, str(tmp_path))
    back = ck.load_packed_checkpoint(str(tmp_path), device=DEV)
    prompt = torch.randint(0, cfg.vocab_size, (2, 19), generator=torch.Generator().manual_seed(4)).to(DEV)
    a = model(prompt, past_key_values=ku.build_paged_cache(model, 2, 24, page_size=16)).logits
    b = back(prompt, past_key_values=ku.build_paged_cache(back, 2, 24, page_size=16)).logits
    assert torch.equal(a, b)
