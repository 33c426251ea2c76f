"""Packed-int4 checkpoint directory: written in the reference's format
(fake_quant/realquant_utils.py:17-141), read back into the decoder, and read by the reference's own
loader where a checkout is present."""
import json
import os

import pytest
import torch

from oracle import ref_shim
from signrot_b200 import checkpoint as ck
from signrot_b200.functional import quantization as qz
from signrot_b200.transformers import kernel_utils as ku


def tiny_model(seed=0):
    cfg = ku.DecoderConfig(hidden_size=256, intermediate_size=768, num_hidden_layers=2, num_attention_heads=2,
                           num_key_value_heads=1, head_dim=128, vocab_size=96)
    return ku.KernelDecoderModel(cfg).random_init_(seed)


@pytest.mark.parametrize("shard", ["5GB", "150KB"])
def test_checkpoint_roundtrip(tmp_path, shard):
    model = tiny_model()
    ck.save_packed_checkpoint(model, str(tmp_path), max_shard_size=shard)
    files = sorted(os.listdir(tmp_path))
    assert "config.json" in files
    sharded = shard != "5GB"
    assert ("model.safetensors.index.json" in files) == sharded
    assert sharded or "model.safetensors" in files
    config, qcfg = ck.read_config(str(tmp_path))
    assert qcfg["quant_method"] == "SignRot" and qcfg["format"] == "packed_int4" and qcfg["w_bits"] == 4
    assert config["hidden_size"] == 256 and config["num_key_value_heads"] == 1

    with ck.Safetensors(str(tmp_path)) as st:
        keys = set(st.keys())
        assert "model.layers.1.mlp.down_proj.had_adj_sign" in keys and "lm_head.weight" in keys
        w = st.get_tensor("model.layers.0.self_attn.q_proj.weight")
        s = st.get_tensor("quantizer.model.layers.0.self_attn.q_proj.scale")
        assert w.dtype == torch.uint8 and w.shape == (256, 128) and s.dtype == torch.float16 and s.shape == (256, 1)
        assert int(st.get_tensor("quantizer.model.layers.0.mlp.up_proj.maxq")) == 7
        assert st.get_tensor("model.layers.0.mlp.down_proj.had_adj_sign").dtype == torch.float16
        first = sorted(set(st.weight_map.values()))[0]
    from safetensors import safe_open
    with safe_open(os.path.join(tmp_path, first), framework="pt") as f:
        assert json.loads(f.metadata()["quantization_config"])["quant_method"] == "SignRot"

    back = ck.load_packed_checkpoint(str(tmp_path), device="cpu")
    want, got = model.state_dict(), back.state_dict()
    assert want.keys() == got.keys()
    for k in want:
        assert torch.equal(want[k], got[k]), k
    at = back.layers[0].self_attn          # loaded models come back with fused projections
    assert at.q_proj.kernel_module.weight.data_ptr() == at.qkv_fused.weight.data_ptr()

    sd, quantizers = ck.load_quantized_weights_with_safetensors(str(tmp_path), dequantize=False)
    name = "model.layers.1.mlp.gate_proj"
    codes = qz.unpack_i4(model.layers[1].mlp.gate_proj.kernel_module.weight)
    assert torch.equal(sd[name + ".weight"], codes.to(torch.float16))
    assert torch.equal(quantizers[name]["scale"], model.layers[1].mlp.gate_proj.kernel_module.weight_scales)
    sd2, _ = ck.load_quantized_weights_with_safetensors(str(tmp_path), dequantize=True)
    assert torch.equal(sd2[name + ".weight"], codes.to(torch.float16) * quantizers[name]["scale"])


def test_loader_rejects_other_formats(tmp_path):
    model = tiny_model()
    ck.save_packed_checkpoint(model, str(tmp_path))
    path = os.path.join(tmp_path, "config.json")
    cfg = json.load(open(path))
    cfg["quantization_config"]["w_asym"] = True
    json.dump(cfg, open(path, "w"))
    with pytest.raises(RuntimeError):
        ck.load_packed_checkpoint(str(tmp_path), device="cpu")


def _edit_qcfg(tmp_path, **changes):
    path = os.path.join(tmp_path, "config.json")
    cfg = json.load(open(path))
    cfg["quantization_config"].update(changes)
    json.dump(cfg, open(path, "w"))


@pytest.mark.parametrize("changes", [dict(rotate_mode="random"), dict(k_bits=16), dict(v_bits=8), dict(k_asym=False),
                                     dict(v_asym=False), dict(int8_down_proj=True), dict(a_bits=8)])
def test_loader_rejects_settings_the_kernels_do_not_run(tmp_path, changes):
    """Every key of the reference's quantization_config (realquant_utils.py:33-49) that would change the arithmetic is
    either honoured or refused; none is ignored."""
    ck.save_packed_checkpoint(tiny_model(), str(tmp_path))
    _edit_qcfg(tmp_path, **changes)
    with pytest.raises(RuntimeError):
        ck.load_packed_checkpoint(str(tmp_path), device="cpu")


def test_bias_and_fp32_rotation_survive_the_round_trip(tmp_path):
    cfg = ku.DecoderConfig(hidden_size=256, intermediate_size=768, num_hidden_layers=2, num_attention_heads=2,
                           num_key_value_heads=1, head_dim=128, vocab_size=96, attention_bias=True, fp32_had=True)
    model = ku.KernelDecoderModel(cfg).random_init_(3)
    g = torch.Generator().manual_seed(0)
    for layer in model.layers:
        for name in ("q_proj", "k_proj", "v_proj"):
            mod = getattr(layer.self_attn, name).kernel_module
            mod.bias.copy_(torch.randn(mod.bias.shape, generator=g).half())
    ck.save_packed_checkpoint(model, str(tmp_path))
    _, qcfg = ck.read_config(str(tmp_path))
    assert qcfg["fp32_had"] is True
    back = ck.load_packed_checkpoint(str(tmp_path), device="cpu", fuse_edges=False)
    assert back.config.attention_bias and back.config.fp32_had
    assert back.layers[1].mlp.down_proj.fp32_had and back.layers[0].self_attn.o_proj.fp32_had
    for a, b in zip(model.layers, back.layers):
        for name in ("q_proj", "k_proj", "v_proj"):
            assert torch.equal(getattr(a.self_attn, name).kernel_module.bias, getattr(b.self_attn, name).kernel_module.bias)


def test_loader_refuses_a_bias_without_a_slot(tmp_path):
    """A bias on a projection the decoder has no bias for (o_proj here) is an error, not a silently dropped tensor."""
    model = tiny_model()
    sd = ck.packed_state_dict(model)
    sd["model.layers.0.self_attn.o_proj.bias"] = torch.zeros(256, dtype=torch.float16)
    ck.save_quantized_weights_with_safetensors(sd, ck.model_config_dict(model.config),
                                               ck.default_quantization_config(model.config), str(tmp_path))
    with pytest.raises(RuntimeError, match="bias"):
        ck.load_packed_checkpoint(str(tmp_path), device="cpu")


@pytest.mark.skipif(not ref_shim.available(), reason="no SignRot checkout on this machine")
def test_reference_loader_reads_our_checkpoint(tmp_path):
    """The reference's `load_quantized_weights_with_safetensors` (realquant_utils.py:266-339) on a
    directory written here: same codes, same scales, same plain tensors."""
    model = tiny_model(1)
    ck.save_packed_checkpoint(model, str(tmp_path), max_shard_size="150KB")
    rq = ref_shim.module("realquant_utils")
    sd, quantizers = rq.load_quantized_weights_with_safetensors(None, str(tmp_path), dequantize=False, device_map="cpu")
    mine, mine_q = ck.load_quantized_weights_with_safetensors(str(tmp_path), dequantize=False)
    assert set(sd.keys()) == set(mine.keys())
    for k in sd:
        assert torch.equal(sd[k], mine[k]), k
    assert set(quantizers.keys()) == set(mine_q.keys())
    for k, wq in quantizers.items():
        assert torch.equal(wq.scale, mine_q[k]["scale"]) and int(wq.maxq) == int(mine_q[k]["maxq"]) == 7
        assert wq.sym and wq.bits == 4
    sd_d, _ = rq.load_quantized_weights_with_safetensors(None, str(tmp_path), dequantize=True, device_map="cpu")
    mine_d, _ = ck.load_quantized_weights_with_safetensors(str(tmp_path), dequantize=True)
    for k in sd_d:
        assert torch.allclose(sd_d[k].float(), mine_d[k].float(), rtol=0, atol=0), k
