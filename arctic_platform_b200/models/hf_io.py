"""Hugging Face weight names <-> the fused layouts of :class:`DecoderLM`.

On disk and on the trainer->sampler sync path weights travel under their Hugging Face
names (``model.layers.N.self_attn.q_proj.weight`` ...), the same contract the reference
keeps for checkpoints (``save_pretrained(..., safe_serialization=True)``,
arctic_platform/common/deepspeed_worker.py:602-636) and for weight sync (310 tensors
for Qwen3-1.7B, arctic_platform/integrations/verl/README.md:96-98).  In memory the
kernels want fused tensors: ``wqkv`` = rows [q | k | v], ``wgu`` = gate and up rows
interleaved (row 2j = gate_j, row 2j+1 = up_j).  This module is the table between the two.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path
from typing import Callable, Dict, Iterator, List, Optional, Tuple

import torch

from .config import DecoderConfig


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return torch.stack([gate, up], dim=1).reshape(2 * gate.shape[0], *gate.shape[1:])


def split_gate_up(wgu: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    return wgu[0::2], wgu[1::2]


# Hugging Face names inside ``linear_attn.`` (split-projection layout) -> attribute of GatedDeltaNet
LINEAR_ATTN_NAMES = ("in_proj_qkv.weight", "in_proj_z.weight", "in_proj_b.weight", "in_proj_a.weight", "conv1d.weight",
                     "dt_bias", "A_log", "norm.weight", "out_proj.weight")
_LINEAR_ATTN_ATTR = {"in_proj_qkv.weight": "in_qkv", "in_proj_z.weight": "in_z", "in_proj_b.weight": "in_b",
                     "in_proj_a.weight": "in_a", "conv1d.weight": "conv_w", "dt_bias": "dt_bias", "A_log": "A_log",
                     "norm.weight": "norm_w", "out_proj.weight": "out_proj"}


def hf_param_names(cfg: DecoderConfig) -> List[str]:
    """Every Hugging Face tensor name of the architecture, in layer order."""
    names = ["model.embed_tokens.weight"]
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        names.append(p + "input_layernorm.weight")
        if cfg.layer_type(i) == "linear_attention":
            names += [p + "linear_attn." + n for n in LINEAR_ATTN_NAMES]
        else:
            names += [p + "self_attn.q_proj.weight", p + "self_attn.k_proj.weight", p + "self_attn.v_proj.weight"]
            if cfg.qk_norm:
                names += [p + "self_attn.q_norm.weight", p + "self_attn.k_norm.weight"]
            names.append(p + "self_attn.o_proj.weight")
        names.append(p + "post_attention_layernorm.weight")
        if cfg.is_moe and cfg.moe_activation == "relu2":
            names += [p + "mlp.gate.weight", p + "mlp.gate.e_score_correction_bias"]
            if cfg.moe_latent_dim:
                names += [p + "mlp.fc1_latent_proj.weight", p + "mlp.fc2_latent_proj.weight"]
            if cfg.shared_expert_intermediate_size > 0:
                names += [p + "mlp.shared_experts.up_proj.weight", p + "mlp.shared_experts.down_proj.weight"]
            for e in range(cfg.num_experts):
                names += [p + f"mlp.experts.{e}.up_proj.weight", p + f"mlp.experts.{e}.down_proj.weight"]
        elif cfg.is_moe:
            names.append(p + "mlp.gate.weight")
            if cfg.shared_expert_intermediate_size > 0:
                names += [p + "mlp.shared_expert.gate_proj.weight", p + "mlp.shared_expert.up_proj.weight",
                          p + "mlp.shared_expert.down_proj.weight", p + "mlp.shared_expert_gate.weight"]
            for e in range(cfg.num_experts):
                names += [p + f"mlp.experts.{e}.gate_proj.weight", p + f"mlp.experts.{e}.up_proj.weight",
                          p + f"mlp.experts.{e}.down_proj.weight"]
        else:
            names += [p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight", p + "mlp.down_proj.weight"]
    names.append("model.norm.weight")
    if not cfg.tie_word_embeddings:
        names.append("lm_head.weight")
    return names


def _all_experts(moe) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(wgu [E, 2I, H], wdown [E, H, I])`` of one MoE layer.  Under expert parallelism every rank holds ``E / ep``
    experts: the shards are all-gathered over the expert-parallel group (a collective -- every rank of the group
    iterates), layer by layer, and dropped after the layer's tensors were yielded
    (arctic_platform/model/implementations/qwen35/deepspeed_integration.py:262-268 does the same for its sync)."""
    ep = getattr(moe, "ep", None)
    if ep is None or ep.world <= 1:
        return moe.wgu.data, moe.wdown.data
    import torch.distributed as dist
    out = []
    for local in (moe.wgu.data, moe.wdown.data):
        parts = [torch.empty_like(local) for _ in range(ep.world)]
        dist.all_gather(parts, local.contiguous(), group=ep.group)
        out.append(torch.cat(parts, 0))
    return out[0], out[1]


def _local_expert(moe, e: int) -> Optional[int]:
    """Index of global expert ``e`` inside this rank's shard, or ``None`` when another rank owns it."""
    ep = getattr(moe, "ep", None)
    if ep is None or ep.world <= 1:
        return e
    n_local = moe.wgu.shape[0]
    lo = ep.rank * n_local
    return e - lo if lo <= e < lo + n_local else None


def iter_hf_tensors(model) -> Iterator[Tuple[str, torch.Tensor]]:
    """Yields ``(hf_name, tensor)`` views/slices of the fused parameters (no copies except the
    de-interleave of gate/up)."""
    cfg: DecoderConfig = model.cfg
    yield "model.embed_tokens.weight", model.embed.data
    qs, ks = cfg.q_size, cfg.kv_size
    for i, blk in enumerate(model.blocks):
        p = f"model.layers.{i}."
        yield p + "input_layernorm.weight", blk.ln1.data
        if getattr(blk, "linear_attn", None) is not None:
            for n in LINEAR_ATTN_NAMES:
                t = getattr(blk.linear_attn, _LINEAR_ATTN_ATTR[n]).data
                yield p + "linear_attn." + n, (t.unsqueeze(1) if n == "conv1d.weight" else t)
        else:
            w = blk.wqkv.data
            if getattr(blk, "wgate", None) is not None:
                # one projection on disk: per head [query rows | gate rows]
                D, H = cfg.head_dim, w.shape[1]
                both = torch.stack([w[:qs].view(cfg.num_heads, D, H), blk.wgate.data.view(cfg.num_heads, D, H)], 1)
                yield p + "self_attn.q_proj.weight", both.reshape(2 * qs, H)
            else:
                yield p + "self_attn.q_proj.weight", w[:qs]
            yield p + "self_attn.k_proj.weight", w[qs:qs + ks]
            yield p + "self_attn.v_proj.weight", w[qs + ks:]
            if cfg.qk_norm:
                yield p + "self_attn.q_norm.weight", blk.q_norm.data
                yield p + "self_attn.k_norm.weight", blk.k_norm.data
            yield p + "self_attn.o_proj.weight", blk.wo.data
        yield p + "post_attention_layernorm.weight", blk.ln2.data
        if cfg.is_moe and getattr(blk.mlp, "latent", False):
            m = blk.mlp
            yield p + "mlp.gate.weight", m.router.data
            yield p + "mlp.gate.e_score_correction_bias", m.e_score_correction_bias
            if m.fc1 is not None:
                yield p + "mlp.fc1_latent_proj.weight", m.fc1.data
                yield p + "mlp.fc2_latent_proj.weight", m.fc2.data
            if m.shared_wup is not None:
                yield p + "mlp.shared_experts.up_proj.weight", m.shared_wup.data
                yield p + "mlp.shared_experts.down_proj.weight", m.shared_wdown.data
            for e in range(cfg.num_experts):
                yield p + f"mlp.experts.{e}.up_proj.weight", m.wup.data[e]
                yield p + f"mlp.experts.{e}.down_proj.weight", m.wdown.data[e]
        elif cfg.is_moe:
            yield p + "mlp.gate.weight", blk.mlp.router.data
            if blk.mlp.shared_wgu is not None:
                g, u = split_gate_up(blk.mlp.shared_wgu.data)
                yield p + "mlp.shared_expert.gate_proj.weight", g
                yield p + "mlp.shared_expert.up_proj.weight", u
                yield p + "mlp.shared_expert.down_proj.weight", blk.mlp.shared_wdown.data
                yield p + "mlp.shared_expert_gate.weight", blk.mlp.shared_gate.data
            wgu_all, wdown_all = _all_experts(blk.mlp)
            for e in range(cfg.num_experts):
                g, u = split_gate_up(wgu_all[e])
                yield p + f"mlp.experts.{e}.gate_proj.weight", g
                yield p + f"mlp.experts.{e}.up_proj.weight", u
                yield p + f"mlp.experts.{e}.down_proj.weight", wdown_all[e]
            del wgu_all, wdown_all
        else:
            g, u = split_gate_up(blk.wgu.data)
            yield p + "mlp.gate_proj.weight", g
            yield p + "mlp.up_proj.weight", u
            yield p + "mlp.down_proj.weight", blk.wdown.data
    yield "model.norm.weight", model.final_norm.data
    if model.lm_head is not None:
        yield "lm_head.weight", model.lm_head.data


@torch.no_grad()
def load_hf_tensor(model, name: str, tensor: torch.Tensor) -> None:
    """Copies one Hugging Face tensor into its place inside the fused parameters."""
    cfg: DecoderConfig = model.cfg
    qs, ks = cfg.q_size, cfg.kv_size

    def put(dst, src):
        if dst.shape != src.shape:
            raise ValueError(f"{name}: shape {tuple(src.shape)} does not fit {tuple(dst.shape)}")
        dst.copy_(src.to(device=dst.device, dtype=dst.dtype))

    if name == "model.embed_tokens.weight":
        return put(model.embed.data, tensor)
    if name == "model.norm.weight":
        return put(model.final_norm.data, tensor)
    if name == "lm_head.weight":
        if model.lm_head is None:
            return None  # tied: the embedding already carries it
        return put(model.lm_head.data, tensor)
    parts = name.split(".")
    if len(parts) < 5 or parts[0] != "model" or parts[1] != "layers":
        raise KeyError(f"unexpected tensor name {name!r}")
    blk = model.blocks[int(parts[2])]
    rest = ".".join(parts[3:])
    if rest == "input_layernorm.weight":
        return put(blk.ln1.data, tensor)
    if rest == "post_attention_layernorm.weight":
        return put(blk.ln2.data, tensor)
    if parts[3] == "linear_attn":
        sub = ".".join(parts[4:])
        dst = getattr(blk.linear_attn, _LINEAR_ATTN_ATTR[sub]).data
        return put(dst, tensor.squeeze(1) if sub == "conv1d.weight" else tensor)
    if rest == "self_attn.q_proj.weight" and getattr(blk, "wgate", None) is not None:
        D, H = cfg.head_dim, tensor.shape[1]
        both = tensor.view(cfg.num_heads, 2, D, H)
        put(blk.wqkv.data[:qs], both[:, 0].reshape(qs, H))
        return put(blk.wgate.data, both[:, 1].reshape(qs, H))
    if getattr(blk.mlp, "latent", False) and parts[3] == "mlp":
        m, sub = blk.mlp, ".".join(parts[4:])
        plain = {"gate.weight": m.router, "gate.e_score_correction_bias": m.e_score_correction_bias,
                 "fc1_latent_proj.weight": m.fc1, "fc2_latent_proj.weight": m.fc2,
                 "shared_experts.up_proj.weight": m.shared_wup, "shared_experts.down_proj.weight": m.shared_wdown}
        if sub in plain and plain[sub] is not None:
            return put(plain[sub].data, tensor)
        if parts[4] == "experts" and parts[6] in ("up_proj", "down_proj"):
            return put((m.wup if parts[6] == "up_proj" else m.wdown).data[int(parts[5])], tensor)
        raise KeyError(f"unexpected tensor name {name!r}")
    if rest == "mlp.shared_expert.gate_proj.weight":
        return put(blk.mlp.shared_wgu.data[0::2], tensor)
    if rest == "mlp.shared_expert.up_proj.weight":
        return put(blk.mlp.shared_wgu.data[1::2], tensor)
    if rest == "mlp.shared_expert.down_proj.weight":
        return put(blk.mlp.shared_wdown.data, tensor)
    if rest == "mlp.shared_expert_gate.weight":
        return put(blk.mlp.shared_gate.data, tensor)
    if rest == "self_attn.q_proj.weight":
        return put(blk.wqkv.data[:qs], tensor)
    if rest == "self_attn.k_proj.weight":
        return put(blk.wqkv.data[qs:qs + ks], tensor)
    if rest == "self_attn.v_proj.weight":
        return put(blk.wqkv.data[qs + ks:], tensor)
    if rest == "self_attn.q_norm.weight":
        return put(blk.q_norm.data, tensor)
    if rest == "self_attn.k_norm.weight":
        return put(blk.k_norm.data, tensor)
    if rest == "self_attn.o_proj.weight":
        return put(blk.wo.data, tensor)
    if rest == "mlp.gate_proj.weight":
        return put(blk.wgu.data[0::2], tensor)
    if rest == "mlp.up_proj.weight":
        return put(blk.wgu.data[1::2], tensor)
    if rest == "mlp.down_proj.weight":
        return put(blk.wdown.data, tensor)
    if rest == "mlp.gate.weight":
        return put(blk.mlp.router.data, tensor)
    if parts[3] == "mlp" and parts[4] == "experts":
        e = _local_expert(blk.mlp, int(parts[5]))
        which = parts[6]
        if e is None:
            return None                          # expert parallelism: that expert lives on another rank
        if which == "gate_proj":
            return put(blk.mlp.wgu.data[e][0::2], tensor)
        if which == "up_proj":
            return put(blk.mlp.wgu.data[e][1::2], tensor)
        if which == "down_proj":
            return put(blk.mlp.wdown.data[e], tensor)
    raise KeyError(f"unexpected tensor name {name!r}")


# ----------------------------------------------------------------------- safetensors files
_ST_DTYPES = {"F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "I64": torch.int64,
              "I32": torch.int32, "U8": torch.uint8, "F64": torch.float64, "BOOL": torch.bool, "I8": torch.int8,
              "I16": torch.int16}
_ST_NAMES = {v: k for k, v in _ST_DTYPES.items()}


def read_safetensors(path) -> Iterator[Tuple[str, torch.Tensor]]:
    """Streams tensors out of a ``.safetensors`` file through one memory map (no whole-file read)."""
    import numpy as np

    path = Path(path)
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hlen))
    header.pop("__metadata__", None)
    mm = np.memmap(path, dtype=np.uint8, mode="r", offset=8 + hlen)
    for name, info in header.items():
        lo, hi = info["data_offsets"]
        dt = _ST_DTYPES[info["dtype"]]
        buf = torch.from_numpy(np.array(mm[lo:hi]))  # owned copy of just this tensor
        yield name, buf.view(dt).reshape(info["shape"])


def write_safetensors(path, tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None) -> None:
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = metadata
    off = 0
    items = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _ST_NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
        items.append(t)
    hb = json.dumps(header, separators=(",", ":")).encode()
    hb += b" " * ((-len(hb)) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for t in items:
            if t.numel():
                f.write(t.view(torch.uint8).reshape(-1).numpy().tobytes())


def _composite_stream(model, source):
    """A composite (vision + language) checkpoint: language-model tensors under their composite names, then every
    tensor that was carried through from the loaded checkpoint."""
    from .vlm import composite_name
    for name, t in source:
        yield composite_name(name), t
    for name, t in (getattr(model, "passthrough", None) or ()):
        yield name, t


def save_hf_checkpoint(model, out_dir, max_shard_bytes: int = 4 << 30, tensors=None) -> List[str]:
    """Writes ``config.json``, sharded ``model-XXXXX-of-YYYYY.safetensors`` and the index file.
    ``tensors`` overrides the source of ``(name, tensor)`` pairs (e.g. gathered ZeRO shards)."""
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    (out / "config.json").write_text(json.dumps(model.cfg.to_hf_dict(), indent=2))
    shards: List[Dict[str, torch.Tensor]] = [{}]
    size = 0
    source = tensors if tensors is not None else iter_hf_tensors(model)
    if model.cfg.vlm_layout:
        source = _composite_stream(model, source)
    for name, t in source:
        n = t.numel() * t.element_size()
        if size + n > max_shard_bytes and shards[-1]:
            shards.append({})
            size = 0
        shards[-1][name] = t.detach().to("cpu").contiguous().clone()
        size += n
    files, weight_map = [], {}
    for i, sh in enumerate(shards):
        fn = "model.safetensors" if len(shards) == 1 else f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        write_safetensors(out / fn, sh, {"format": "pt"})
        files.append(fn)
        for k in sh:
            weight_map[k] = fn
    if len(shards) > 1:
        (out / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
    copy_tokenizer_files(getattr(model, "source_dir", None), out)
    return files


# ----------------------------------------------------------------------------- plain state dicts in a directory
def get_max_layer_num(state_dict, layer_prefix: str = "model.layers.") -> int:
    """Number of layers named in ``state_dict`` (highest ``<prefix><n>.`` + 1; 0 when there is none).  Works on any
    iterable of names."""
    top = -1
    for key in state_dict:
        if key.startswith(layer_prefix):
            head = key[len(layer_prefix):].split(".", 1)[0]
            if head.isdigit():
                top = max(top, int(head))
    return top + 1


def safetensors_keys(path) -> List[str]:
    """Tensor names of one ``.safetensors`` file, from its header only."""
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hlen))
    return [k for k in header if k != "__metadata__"]


def load_state_dict_keys(save_dir) -> List[str]:
    """Names of every tensor in the ``*.safetensors`` files of a directory; no tensor data is read."""
    return [k for p in sorted(Path(save_dir).glob("*.safetensors")) for k in safetensors_keys(p)]


def load_state_dict(save_dir) -> Dict[str, torch.Tensor]:
    """Every tensor of the ``*.safetensors`` files of a directory, on the CPU."""
    return {k: t for p in sorted(Path(save_dir).glob("*.safetensors")) for k, t in read_safetensors(p)}


def save_state_dict(state_dict: Dict[str, torch.Tensor], save_dir, save_format: str = "safetensors",
                    save_sharded: bool = True, max_shard_bytes: int = 5 << 30) -> List[str]:
    """Writes a name -> tensor mapping as ``model.safetensors`` (or ``model-XXXXX-of-YYYYY.safetensors`` plus
    ``model.safetensors.index.json`` when it exceeds ``max_shard_bytes`` and ``save_sharded``); ``save_format="torch"``
    writes ``pytorch_model.bin``.  Returns the file names.  Same call as
    arctic_platform/model/implementations/qwen35/weights.py:59-103."""
    out = Path(save_dir)
    out.mkdir(parents=True, exist_ok=True)
    if save_format == "torch":
        torch.save({k: v.detach().to("cpu") for k, v in state_dict.items()}, out / "pytorch_model.bin")
        return ["pytorch_model.bin"]
    if save_format != "safetensors":
        raise ValueError(f"save_format {save_format!r}: expected 'safetensors' or 'torch'")
    shards: List[Dict[str, torch.Tensor]] = [{}]
    size = 0
    for name, t in state_dict.items():
        n = t.numel() * t.element_size()
        if save_sharded and size + n > max_shard_bytes and shards[-1]:
            shards.append({})
            size = 0
        shards[-1][name] = t.detach().to("cpu").contiguous()
        size += n
    files, weight_map, total = [], {}, 0
    for i, sh in enumerate(shards):
        fn = "model.safetensors" if len(shards) == 1 else f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        write_safetensors(out / fn, sh, {"format": "pt"})
        files.append(fn)
        for k, t in sh.items():
            weight_map[k] = fn
            total += t.numel() * t.element_size()
    if len(shards) > 1:
        (out / "model.safetensors.index.json").write_text(json.dumps({"metadata": {"total_size": total},
                                                                       "weight_map": weight_map}))
    return files


TOKENIZER_FILES = ("tokenizer.json", "tokenizer_config.json", "tokenizer.model", "special_tokens_map.json", "vocab.json",
                   "merges.txt", "added_tokens.json", "generation_config.json", "chat_template.jinja", "chat_template.json")


def copy_tokenizer_files(source_dir, out_dir) -> List[str]:
    """An exported checkpoint is loadable on its own: the tokenizer, generation config and chat template of the
    checkpoint the model was loaded from travel with the new weights."""
    import shutil
    if not source_dir:
        return []
    src, dst, done = Path(source_dir), Path(out_dir), []
    if not src.is_dir() or src.resolve() == dst.resolve():
        return []
    for name in TOKENIZER_FILES:
        if (src / name).is_file():
            shutil.copy2(src / name, dst / name)
            done.append(name)
    return done


def load_hf_checkpoint(model, ckpt_dir, strict: bool = True) -> int:
    """Loads every ``*.safetensors`` under ``ckpt_dir`` into ``model``; returns the tensor count."""
    d = Path(ckpt_dir)
    files = sorted(d.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors files in {d}")
    from .vlm import PassthroughTensors, text_name
    expected = set(hf_param_names(model.cfg))
    seen = set()
    for f in files:
        for raw, t in read_safetensors(f):
            name = text_name(raw)
            if name is None:                  # vision tower / extra heads of a composite checkpoint: kept, not trained
                if getattr(model, "passthrough", None) is None:
                    model.passthrough = PassthroughTensors()
                model.passthrough.add(raw, t)
                continue
            if name not in expected:
                if strict and not (name == "lm_head.weight" and model.lm_head is None):
                    raise KeyError(f"{f.name}: unexpected tensor {name!r}")
                continue
            load_hf_tensor(model, name, t)
            seen.add(name)
    if strict and seen != expected:
        raise KeyError(f"checkpoint is missing {sorted(expected - seen)[:5]} ...")
    return len(seen)
