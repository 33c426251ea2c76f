"""Packed-int4 checkpoints in the reference's on-disk format
(fake_quant/realquant_utils.py:17-339; key mapping of the deployment model:
e2e/quantized_llama/modeling_llama.py:253-263).

Layout of a checkpoint directory:

  config.json                     the model config plus a `quantization_config` block
                                  (`quant_method: SignRot`, `format: packed_int4`, bit widths, ...)
  model.safetensors               or `model-0000x-of-0000y.safetensors` shards of at most 5 GB with
  model.safetensors.index.json    `{"metadata": ..., "weight_map": {tensor name: file}}`

Tensors, named as in a Hugging Face Llama state dict:

  <linear>.weight                 uint8 [N, K/2]: two's-complement int4 codes, element 2j in the low
                                  nibble of byte j (`pack_i4`), for every quantized linear
  quantizer.<linear>.scale        fp16 [N, 1] per-channel weight scale
  quantizer.<linear>.maxq         the quantizer's maxq (7 for symmetric int4)
  <linear>.had_adj_sign           +-1 SignRot adjustment of an online-rotated linear (stored as fp16,
                                  as the reference's writer casts every non-packed tensor to half)
  everything else                 fp16 (embedding, lm_head)

The first file's safetensors metadata carries the `quantization_config` JSON.  This module writes and
reads that format for the self-contained decoder of `transformers/kernel_utils.py`; the tensors go
straight into `Linear4bit.weight / weight_scales` and `OnlineHadamard.had_adj_sign` (no unpacking:
the kernels consume the packed bytes)."""
from __future__ import annotations

import json
import os
from contextlib import ExitStack

import torch

PROJECTIONS = (("self_attn", "q_proj"), ("self_attn", "k_proj"), ("self_attn", "v_proj"), ("self_attn", "o_proj"),
               ("mlp", "gate_proj"), ("mlp", "up_proj"), ("mlp", "down_proj"))


def default_quantization_config(cfg) -> dict:
    """The `quantization_config` block the reference's writer emits (realquant_utils.py:32-50), filled
    for what this package runs: W4 symmetric per-channel RTN weights, A4 per-token activations, int4
    asymmetric K/V per head vector, online Hadamard rotations with the SignRot adjustment on down_proj."""
    return {
        "quant_method": "SignRot", "w_quantizer": "rtn",
        "w_bits": 4, "w_asym": False, "w_groupsize": -1, "w_clip": False, "w_perchannel": True,
        "a_bits": 4, "a_asym": bool(cfg.a_asym), "a_groupsize": -1, "a_clip_ratio": float(cfg.a_clip_ratio),
        "k_bits": 4, "k_asym": True, "k_groupsize": cfg.head_dim, "k_clip_ratio": 1.0,
        "v_bits": 4, "v_asym": True, "v_groupsize": cfg.head_dim, "v_clip_ratio": 1.0,
        "format": "packed_int4",
        "rotate": True, "rotate_mode": "hadamard", "fp32_had": bool(getattr(cfg, "fp32_had", False)),
        "adj_layers": ["down_proj"] if cfg.had_adj else [],
        "int8_down_proj": False,
    }


def model_config_dict(cfg) -> dict:
    """Hugging Face Llama config keys of a DecoderConfig."""
    return {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size,
        "num_hidden_layers": cfg.num_hidden_layers, "num_attention_heads": cfg.num_attention_heads,
        "num_key_value_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "vocab_size": cfg.vocab_size,
        "rms_norm_eps": cfg.rms_norm_eps, "rope_theta": cfg.rope_theta, "torch_dtype": "float16",
    }


def packed_state_dict(model) -> dict:
    """The tensors of a dense `KernelDecoderModel` under the reference's names (CPU tensors)."""
    if model.config.num_local_experts:
        raise NotImplementedError("sparse (MoE) stacks are not covered by the packed checkpoint writer")
    out = {"model.embed_tokens.weight": model.embed_tokens.weight.detach().to(torch.float16).cpu().contiguous(),
           "lm_head.weight": model.lm_head.weight.detach().to(torch.float16).cpu().contiguous()}
    for i, layer in enumerate(model.layers):
        for parent, name in PROJECTIONS:
            lin = getattr(getattr(layer, parent), name)
            key = f"model.layers.{i}.{parent}.{name}"
            mod = lin.kernel_module
            out[key + ".weight"] = mod.weight.detach().cpu().contiguous()
            out[f"quantizer.{key}.scale"] = mod.weight_scales.detach().to(torch.float16).cpu().reshape(-1, 1).contiguous()
            out[f"quantizer.{key}.maxq"] = torch.tensor(7)
            if mod.bias is not None:
                out[key + ".bias"] = mod.bias.detach().to(torch.float16).cpu().contiguous()
            had = lin.kernel_hadamard
            if had is not None and had.had_adj_sign is not None:
                out[key + ".had_adj_sign"] = had.had_adj_sign.detach().to(torch.float16).cpu().contiguous()
    return out


def save_quantized_weights_with_safetensors(state_dict: dict, config: dict, quantization_config: dict, save_dir: str,
                                            max_shard_size="5GB") -> None:
    """Writes `state_dict` (already packed, see `packed_state_dict`) as the reference's writer does
    (realquant_utils.py:89-141): shards of `max_shard_size`, metadata on the first file, index
    file when sharded, config.json with the quantization block."""
    from safetensors.torch import save_file
    from huggingface_hub import split_torch_state_dict_into_shards
    os.makedirs(save_dir, exist_ok=True)
    metadata = {"quantization_config": json.dumps(quantization_config)}
    split = split_torch_state_dict_into_shards(state_dict, max_shard_size=max_shard_size,
                                               filename_pattern="model{suffix}.safetensors")
    first = True
    for filename, names in split.filename_to_tensors.items():
        shard = {n: state_dict[n] for n in names}
        save_file(shard, os.path.join(save_dir, filename), metadata=metadata if first else None)
        first = False
    if split.is_sharded:
        index = {"metadata": getattr(split, "metadata", {}), "weight_map": split.tensor_to_filename}
        with open(os.path.join(save_dir, "model.safetensors.index.json"), "w") as f:
            json.dump(index, f, indent=2)
    with open(os.path.join(save_dir, "config.json"), "w") as f:
        json.dump({**config, "quantization_config": quantization_config}, f, indent=2)


def save_packed_checkpoint(model, save_dir: str, max_shard_size="5GB") -> None:
    """A dense `KernelDecoderModel` -> checkpoint directory."""
    cfg = model.config
    save_quantized_weights_with_safetensors(packed_state_dict(model), model_config_dict(cfg),
                                            default_quantization_config(cfg), save_dir, max_shard_size)


class Safetensors:
    """Read access to a single-file or sharded checkpoint (realquant_utils.py:185-258), tensors
    materialised on `device`."""

    def __init__(self, load_path: str, device="cpu"):
        from safetensors import safe_open
        self.load_path = load_path
        self.device = str(torch.device(device))
        index_path = os.path.join(load_path, "model.safetensors.index.json")
        self.metadata = {}
        self.weight_map = {}
        if os.path.exists(index_path):
            with open(index_path) as f:
                index = json.load(f)
            self.metadata = index.get("metadata", {})
            self.weight_map = dict(index["weight_map"])
        else:
            with safe_open(os.path.join(load_path, "model.safetensors"), framework="pt") as f:
                self.metadata = f.metadata() or {}
                for key in f.keys():
                    self.weight_map[key] = "model.safetensors"
        self._open = safe_open
        self._files = {}
        self._stack = None

    def keys(self):
        return self.weight_map.keys()

    def get_tensor(self, key: str) -> torch.Tensor:
        if key not in self.weight_map:
            raise KeyError(f"Key {key} not found in safetensors.")
        return self._files[self.weight_map[key]].get_tensor(key)

    def __enter__(self):
        self._stack = ExitStack()
        for filename in sorted(set(self.weight_map.values())):
            handle = self._open(os.path.join(self.load_path, filename), framework="pt", device=self.device)
            self._files[filename] = self._stack.enter_context(handle)
        return self

    def __exit__(self, exc_type, exc_value, traceback):
        self._stack.close()
        self._files = {}


def read_config(load_path: str):
    with open(os.path.join(load_path, "config.json")) as f:
        config = json.load(f)
    return config, config.get("quantization_config", {})


@torch.no_grad()
def load_quantized_weights_with_safetensors(load_path: str, dequantize=False, device="cpu", dtype=torch.float16):
    """What the reference's loader returns (realquant_utils.py:266-339): `(state_dict, quantizers)`
    with the packed weights unpacked to integer codes (or dequantized `codes * scale`) in `dtype`, and
    per linear a dict of its `scale` / `zero` / `maxq` tensors."""
    from .functional.quantization import unpack_i4
    state_dict, quantizers = {}, {}
    with Safetensors(load_path, device) as st:
        plain = []
        for k in st.keys():
            if not k.startswith("quantizer."):
                plain.append(k)
                continue
            _, *atoms, kind = k.split(".")
            quantizers.setdefault(".".join(atoms), {})[kind] = st.get_tensor(k)
        for k in plain:
            v = st.get_tensor(k)
            if k.endswith(".weight") and k.rsplit(".", 1)[0] in quantizers:
                v = unpack_i4(v).to(torch.int8)
                if dequantize:
                    v = v.to(dtype) * quantizers[k.rsplit(".", 1)[0]]["scale"].to(v.device, dtype)
            state_dict[k] = v.to(dtype)
    return state_dict, quantizers


@torch.no_grad()
def load_packed_checkpoint(load_path: str, device="cuda", fuse_edges=True):
    """Checkpoint directory -> `KernelDecoderModel` on `device`, packed bytes copied as they are."""
    from .transformers import kernel_utils as ku
    config, qcfg = read_config(load_path)
    if qcfg.get("format", "packed_int4") != "packed_int4" or qcfg.get("w_bits", 4) != 4 or qcfg.get("w_asym", False):
        raise RuntimeError("only packed symmetric int4 checkpoints are supported")
    if qcfg.get("a_bits", 4) != 4:
        raise RuntimeError("the kernels quantize activations to 4 bits")
    # Settings the model would otherwise run differently from what the checkpoint was calibrated for
    # (the keys of realquant_utils.py:33-49): the online rotations are Hadamard, the cache is 4-bit asymmetric
    # per head vector, down_proj takes 4-bit activations.
    if qcfg.get("rotate_mode", "hadamard") != "hadamard":
        raise RuntimeError(f"rotate_mode {qcfg['rotate_mode']!r} is not supported: the online rotations are Hadamard")
    for which in ("k", "v"):
        if qcfg.get(f"{which}_bits", 4) != 4 or not qcfg.get(f"{which}_asym", True):
            raise RuntimeError(f"the KV cache stores asymmetric 4-bit codes; the checkpoint asks for "
                               f"{which}_bits={qcfg.get(f'{which}_bits')}, {which}_asym={qcfg.get(f'{which}_asym')}")
    if qcfg.get("int8_down_proj", False):
        raise RuntimeError("int8_down_proj checkpoints are not supported")
    heads = config["num_attention_heads"]
    with Safetensors(load_path, "cpu") as st:
        all_keys = set(st.keys())
    bias_keys = {k for k in all_keys if k.endswith(".bias")}
    qkv_bias = {f"model.layers.{i}.self_attn.{n}.bias" for i in range(config["num_hidden_layers"])
                for n in ("q_proj", "k_proj", "v_proj")}
    if bias_keys - qkv_bias:
        raise RuntimeError(f"bias on a projection that has no bias slot: {sorted(bias_keys - qkv_bias)[0]}")
    if bias_keys and bias_keys != qkv_bias:
        raise RuntimeError("q/k/v biases must be present for every layer or for none")
    cfg = ku.DecoderConfig(
        hidden_size=config["hidden_size"], intermediate_size=config["intermediate_size"],
        num_hidden_layers=config["num_hidden_layers"], num_attention_heads=heads,
        num_key_value_heads=config.get("num_key_value_heads", heads),
        head_dim=config.get("head_dim") or config["hidden_size"] // heads, vocab_size=config["vocab_size"],
        rms_norm_eps=config.get("rms_norm_eps", 1e-5), rope_theta=config.get("rope_theta", 10000.0),
        a_asym=bool(qcfg.get("a_asym", False)), a_clip_ratio=float(qcfg.get("a_clip_ratio", 1.0)),
        had_adj="down_proj" in (qcfg.get("adj_layers") or []), fp32_had=bool(qcfg.get("fp32_had", False)),
        attention_bias=bool(bias_keys), fuse_edges=fuse_edges)
    with torch.device(device):
        model = ku.KernelDecoderModel(cfg)
    model = model.to(device)
    with Safetensors(load_path, device) as st:
        keys = set(st.keys())
        model.embed_tokens.weight.copy_(st.get_tensor("model.embed_tokens.weight"))
        head = "lm_head.weight" if "lm_head.weight" in keys else "model.embed_tokens.weight"   # tied embeddings
        model.lm_head.weight.copy_(st.get_tensor(head))
        for i, layer in enumerate(model.layers):
            for parent, name in PROJECTIONS:
                lin = getattr(getattr(layer, parent), name)
                key = f"model.layers.{i}.{parent}.{name}"
                mod = lin.kernel_module
                w = st.get_tensor(key + ".weight")
                if w.dtype != torch.uint8 or w.shape != mod.weight.shape:
                    raise RuntimeError(f"{key}.weight: expected packed uint8 {tuple(mod.weight.shape)}, got {w.dtype} {tuple(w.shape)}")
                mod.weight.copy_(w)
                mod.weight_scales = st.get_tensor(f"quantizer.{key}.scale").to(torch.float16).reshape(-1, 1).contiguous()
                if key + ".bias" in keys:
                    mod.bias.copy_(st.get_tensor(key + ".bias").to(torch.float16))
                sign_key = key + ".had_adj_sign"
                had = lin.kernel_hadamard
                if sign_key in keys:
                    if had is None or had.had_adj_sign is None:
                        raise RuntimeError(f"{sign_key}: this linear has no sign-adjusted rotation")
                    had.had_adj_sign.copy_(st.get_tensor(sign_key).to(torch.int8))
    return model.fuse_projections_()
