"""Synthetic stand-ins for the models and SquareQ slabs the streaming path is measured on.

No checkpoint, SquareQ slab or dataset ships with the reference, so the tests,
the smoke check and the benchmark build models with the published *shapes* and
fill SquareQ ``.fpk`` payloads with seeded synthetic values:

* int8 weights uniform on [-127, 127];
* fp32 per-output-channel scales ``exp(randn * 0.5 + ln 0.01)``;
* zero points 0 (symmetric quantisation), fp32;
* fp32 biases ``randn * 0.02``.

The ``.fpk`` container is the one the reference loads with ``torch.load``
(``src/stagehand/registry.py:339-387`` reads ``payload["manifest"]["layers"]``
entries ``{name, out, inp, padded_in, has_bias}``; ``src/stagehand/scheduler.py:603-629``
reads ``payload["layers"][name]`` dicts ``{qweight, scale, zero_point, bias}``).

Every projection is a :class:`GainLinear`: an ``nn.Linear`` whose output is
multiplied by a constant so activations stay O(1) with these weight magnitudes;
parameter names and shapes are those of ``nn.Linear``.
"""
from __future__ import annotations

import math
import re
from pathlib import Path

import torch
import torch.nn.functional as F
from torch import nn

__all__ = [
    "GainLinear",
    "TinyBlockModel",
    "FluxShapedDiT",
    "MistralShapedEncoder",
    "EncoderPlusDiT",
    "LoraLinear",
    "VideoShapedDiT",
    "write_sharded_safetensors",
    "synth_squareq_layer",
    "write_squareq_fpk",
    "BLOCK_PATTERNS",
]

# E|q| statistics of the synthetic weights: std(q) for uniform[-127,127] is ~73.3 and
# E[scale^2]^(1/2) = 0.01 * exp(0.25) for lognormal(ln 0.01, 0.5).
_SYNTH_WEIGHT_STD = 73.32 * 0.01 * math.exp(0.25)


class GainLinear(nn.Linear):
    """``nn.Linear`` followed by a fixed scalar gain of ``1 / (w_std * sqrt(in))``."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None) -> None:
        super().__init__(in_features, out_features, bias=bias, device=device, dtype=dtype)
        self.gain = 1.0 / (_SYNTH_WEIGHT_STD * math.sqrt(in_features))

    def reset_parameters(self) -> None:  # values always come from the slab; skip the costly init
        return

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.linear(x, self.weight, self.bias) * self.gain


def _sdpa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """[B, H, T, D] attention -> [B, T, H*D]."""
    out = F.scaled_dot_product_attention(q, k, v)
    b, h, t, d = out.shape
    return out.transpose(1, 2).reshape(b, t, h * d)


def _heads(x: torch.Tensor, n_heads: int) -> torch.Tensor:
    b, t, hd = x.shape
    return x.view(b, t, n_heads, hd // n_heads).transpose(1, 2)


# ── config 1: plain pre-norm transformer blocks ──────────────────────────


class _PlainBlock(nn.Module):
    def __init__(self, hidden: int, heads: int, mlp: int, device=None, dtype=None) -> None:
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        self.heads = heads
        self.norm1 = nn.LayerNorm(hidden, **kw)
        self.qkv = GainLinear(hidden, 3 * hidden, **kw)
        self.out = GainLinear(hidden, hidden, **kw)
        self.norm2 = nn.LayerNorm(hidden, **kw)
        self.fc1 = GainLinear(hidden, mlp, **kw)
        self.fc2 = GainLinear(mlp, hidden, **kw)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        q, k, v = self.qkv(self.norm1(x)).chunk(3, dim=-1)
        x = x + self.out(_sdpa(_heads(q, self.heads), _heads(k, self.heads), _heads(v, self.heads)))
        return x + self.fc2(F.gelu(self.fc1(self.norm2(x))))


class TinyBlockModel(nn.Module):
    """``blocks.{i}`` = LayerNorm, qkv, out, LayerNorm, fc1, fc2 (the CPU block-mode configuration).

    Defaults are the named configuration: 4 blocks, hidden 1024, 16 heads, MLP 4096.
    """

    def __init__(self, n_blocks: int = 4, hidden: int = 1024, heads: int = 16, mlp: int = 4096,
                 device=None, dtype=None) -> None:
        super().__init__()
        self.blocks = nn.ModuleList(_PlainBlock(hidden, heads, mlp, device, dtype) for _ in range(n_blocks))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        for block in self.blocks:
            x = block(x)
        return x


# ── config 2: Flux-1-dev-shaped DiT ──────────────────────────────────────


def _modulate(x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return F.layer_norm(x, x.shape[-1:]) * (1 + scale.unsqueeze(1)) + shift.unsqueeze(1)


class _StreamHalf(nn.Module):
    """One stream (image or text) of a double-stream block."""

    def __init__(self, hidden: int, heads: int, mlp: int, device=None, dtype=None) -> None:
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        self.mod = GainLinear(hidden, 6 * hidden, **kw)
        self.qkv = GainLinear(hidden, 3 * hidden, **kw)
        self.q_norm = nn.RMSNorm(hidden // heads, **kw)
        self.k_norm = nn.RMSNorm(hidden // heads, **kw)
        self.proj = GainLinear(hidden, hidden, **kw)
        self.mlp_in = GainLinear(hidden, mlp, **kw)
        self.mlp_out = GainLinear(mlp, hidden, **kw)


class _DoubleStreamBlock(nn.Module):
    def __init__(self, hidden: int, heads: int, mlp: int, device=None, dtype=None) -> None:
        super().__init__()
        self.heads = heads
        self.img = _StreamHalf(hidden, heads, mlp, device, dtype)
        self.txt = _StreamHalf(hidden, heads, mlp, device, dtype)

    def _qkv(self, half: _StreamHalf, x: torch.Tensor, mod: tuple[torch.Tensor, ...]):
        q, k, v = half.qkv(_modulate(x, mod[0], mod[1])).chunk(3, dim=-1)
        q, k, v = _heads(q, self.heads), _heads(k, self.heads), _heads(v, self.heads)
        return half.q_norm(q), half.k_norm(k), v

    @staticmethod
    def _finish(half: _StreamHalf, x: torch.Tensor, attn: torch.Tensor, mod: tuple[torch.Tensor, ...]) -> torch.Tensor:
        x = x + mod[2].unsqueeze(1) * half.proj(attn)
        h = half.mlp_out(F.gelu(half.mlp_in(_modulate(x, mod[3], mod[4])), approximate="tanh"))
        return x + mod[5].unsqueeze(1) * h

    def forward(self, img: torch.Tensor, txt: torch.Tensor, vec: torch.Tensor):
        act = F.silu(vec)
        img_mod = self.img.mod(act).chunk(6, dim=-1)
        txt_mod = self.txt.mod(act).chunk(6, dim=-1)
        iq, ik, iv = self._qkv(self.img, img, img_mod)
        tq, tk, tv = self._qkv(self.txt, txt, txt_mod)
        attn = _sdpa(torch.cat((tq, iq), dim=2), torch.cat((tk, ik), dim=2), torch.cat((tv, iv), dim=2))
        n_txt = txt.shape[1]
        img = self._finish(self.img, img, attn[:, n_txt:], img_mod)
        txt = self._finish(self.txt, txt, attn[:, :n_txt], txt_mod)
        return img, txt


class _SingleStreamBlock(nn.Module):
    def __init__(self, hidden: int, heads: int, mlp: int, device=None, dtype=None) -> None:
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        self.heads, self.hidden, self.mlp = heads, hidden, mlp
        self.mod = GainLinear(hidden, 3 * hidden, **kw)
        self.lin1 = GainLinear(hidden, 3 * hidden + mlp, **kw)
        self.q_norm = nn.RMSNorm(hidden // heads, **kw)
        self.k_norm = nn.RMSNorm(hidden // heads, **kw)
        self.lin2 = GainLinear(hidden + mlp, hidden, **kw)

    def forward(self, x: torch.Tensor, vec: torch.Tensor) -> torch.Tensor:
        shift, scale, gate = self.mod(F.silu(vec)).chunk(3, dim=-1)
        qkv, mlp = self.lin1(_modulate(x, shift, scale)).split((3 * self.hidden, self.mlp), dim=-1)
        q, k, v = qkv.chunk(3, dim=-1)
        attn = _sdpa(self.q_norm(_heads(q, self.heads)), self.k_norm(_heads(k, self.heads)), _heads(v, self.heads))
        out = self.lin2(torch.cat((attn, F.gelu(mlp, approximate="tanh")), dim=-1))
        return x + gate.unsqueeze(1) * out


class FluxShapedDiT(nn.Module):
    """19 double-stream + 38 single-stream blocks, hidden 3072, 24 heads, MLP ratio 4.

    Per double block (two streams): mod 18432x3072, qkv 9216x3072, proj 3072x3072,
    mlp 12288x3072 and 3072x12288 -> 339.7 M weights.  Per single block: lin1
    21504x3072, lin2 3072x15360, mod 9216x3072 -> 141.6 M weights.  Positional
    embeddings and the input/output projections are left out: only the streamed
    blocks matter here.
    """

    def __init__(self, n_double: int = 19, n_single: int = 38, hidden: int = 3072, heads: int = 24,
                 mlp_ratio: int = 4, device=None, dtype=None) -> None:
        super().__init__()
        mlp = hidden * mlp_ratio
        self.hidden = hidden
        self.double_blocks = nn.ModuleList(
            _DoubleStreamBlock(hidden, heads, mlp, device, dtype) for _ in range(n_double))
        self.single_blocks = nn.ModuleList(
            _SingleStreamBlock(hidden, heads, mlp, device, dtype) for _ in range(n_single))

    def forward(self, img: torch.Tensor, txt: torch.Tensor, vec: torch.Tensor) -> torch.Tensor:
        for block in self.double_blocks:
            img, txt = block(img, txt, vec)
        x = torch.cat((txt, img), dim=1)
        for block in self.single_blocks:
            x = block(x, vec)
        return x[:, txt.shape[1]:]


# ── config 5: Mistral-24B-shaped text encoder ────────────────────────────


class _GqaLayer(nn.Module):
    def __init__(self, hidden: int, q_heads: int, kv_heads: int, head_dim: int, ffn: int,
                 device=None, dtype=None) -> None:
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        self.q_heads, self.kv_heads = q_heads, kv_heads
        self.input_norm = nn.RMSNorm(hidden, **kw)
        self.q_proj = GainLinear(hidden, q_heads * head_dim, bias=False, **kw)
        self.k_proj = GainLinear(hidden, kv_heads * head_dim, bias=False, **kw)
        self.v_proj = GainLinear(hidden, kv_heads * head_dim, bias=False, **kw)
        self.o_proj = GainLinear(q_heads * head_dim, hidden, bias=False, **kw)
        self.post_norm = nn.RMSNorm(hidden, **kw)
        self.gate_proj = GainLinear(hidden, ffn, bias=False, **kw)
        self.up_proj = GainLinear(hidden, ffn, bias=False, **kw)
        self.down_proj = GainLinear(ffn, hidden, bias=False, **kw)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = self.input_norm(x)
        q = _heads(self.q_proj(h), self.q_heads)
        k = _heads(self.k_proj(h), self.kv_heads)
        v = _heads(self.v_proj(h), self.kv_heads)
        rep = self.q_heads // self.kv_heads
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
        x = x + self.o_proj(_sdpa(q, k, v))
        h = self.post_norm(x)
        return x + self.down_proj(F.silu(self.gate_proj(h)) * self.up_proj(h))


class MistralShapedEncoder(nn.Module):
    """40 layers, hidden 5120, 32 query / 8 kv heads of 128, FFN 32768 (555.7 M weights per layer)."""

    def __init__(self, n_layers: int = 40, hidden: int = 5120, q_heads: int = 32, kv_heads: int = 8,
                 head_dim: int = 128, ffn: int = 32768, device=None, dtype=None) -> None:
        super().__init__()
        self.hidden = hidden
        self.layers = nn.ModuleList(
            _GqaLayer(hidden, q_heads, kv_heads, head_dim, ffn, device, dtype) for _ in range(n_layers))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        for layer in self.layers:
            x = layer(x)
        return x


# ── config 3: bf16 video-DiT-shaped blocks with rank-r adapters (forward + backward) ──────────


class LoraLinear(nn.Module):
    """A frozen bias-free projection (``base.weight``, streamed from a file) plus a trainable rank-r adapter.

    ``lora_a`` / ``lora_b`` require gradients, so the registry keeps them module-owned
    (reference ``src/stagehand/registry.py:648-650``): they are staged fresh at every load
    and their gradients are kept at eviction.
    """

    def __init__(self, in_features: int, out_features: int, rank: int, device=None, dtype=None) -> None:
        super().__init__()
        self.base = nn.Linear(in_features, out_features, bias=False, device=device, dtype=dtype)
        self.lora_a = nn.Parameter(torch.empty(rank, in_features, device=device, dtype=dtype))
        self.lora_b = nn.Parameter(torch.empty(out_features, rank, device=device, dtype=dtype))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.base(x) + F.linear(F.linear(x, self.lora_a), self.lora_b)


class _VideoDiTBlock(nn.Module):
    """Self-attention, cross-attention to a text context and a GELU feed-forward, all pre-norm."""

    def __init__(self, hidden: int, heads: int, ffn: int, rank: int, device=None, dtype=None) -> None:
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        self.heads = heads
        self.norm1 = nn.RMSNorm(hidden, **kw)
        self.attn_q, self.attn_k, self.attn_v, self.attn_o = (LoraLinear(hidden, hidden, rank, **kw) for _ in range(4))
        self.norm2 = nn.RMSNorm(hidden, **kw)
        self.cross_q, self.cross_k, self.cross_v, self.cross_o = (LoraLinear(hidden, hidden, rank, **kw) for _ in range(4))
        self.norm3 = nn.RMSNorm(hidden, **kw)
        self.fc1 = nn.Linear(hidden, ffn, bias=False, **kw)
        self.fc2 = nn.Linear(ffn, hidden, bias=False, **kw)

    def forward(self, x: torch.Tensor, context: torch.Tensor) -> torch.Tensor:
        n = self.heads
        h = self.norm1(x)
        x = x + self.attn_o(_sdpa(_heads(self.attn_q(h), n), _heads(self.attn_k(h), n), _heads(self.attn_v(h), n)))
        h = self.norm2(x)
        x = x + self.cross_o(_sdpa(_heads(self.cross_q(h), n), _heads(self.cross_k(context), n),
                                   _heads(self.cross_v(context), n)))
        return x + self.fc2(F.gelu(self.fc1(self.norm3(x))))


class VideoShapedDiT(nn.Module):
    """48 blocks, hidden 4096, 32 heads, FFN 16384, rank-32 adapters on the eight attention projections.

    With these dimensions a block holds 8 x 4096^2 + 2 x 4096 x 16384 = 268.4 M frozen weights
    (12.9 G in 48 blocks, 25.8 GB in bf16) and 2.1 M trainable adapter weights.  With
    ``checkpoint_blocks`` every block runs under activation checkpointing, the way the
    reference's training case study runs (its blocks are recomputed during backward).
    """

    def __init__(self, n_blocks: int = 48, hidden: int = 4096, heads: int = 32, ffn: int = 16384, rank: int = 32,
                 checkpoint_blocks: bool = True, device=None, dtype=None) -> None:
        super().__init__()
        self.checkpoint_blocks = checkpoint_blocks
        self.blocks = nn.ModuleList(_VideoDiTBlock(hidden, heads, ffn, rank, device, dtype) for _ in range(n_blocks))

    def init_adapters(self, seed: int = 0, std: float = 0.02) -> None:
        """Real storage and seeded values for the adapters (also when the model was built on ``meta``)."""
        g = torch.Generator().manual_seed(seed)
        for module in self.modules():
            if isinstance(module, LoraLinear):
                for name in ("lora_a", "lora_b"):
                    old = getattr(module, name)
                    value = (torch.randn(old.shape, generator=g) * std).to(old.dtype)
                    setattr(module, name, nn.Parameter(value, requires_grad=True))

    def forward(self, x: torch.Tensor, context: torch.Tensor) -> torch.Tensor:
        from torch.utils.checkpoint import checkpoint

        for block in self.blocks:
            if self.checkpoint_blocks and torch.is_grad_enabled():
                x = checkpoint(block, x, context, use_reentrant=False)
            else:
                x = block(x, context)
        return x


_SAFETENSORS_DTYPES = {torch.bfloat16: "BF16", torch.float16: "F16", torch.float32: "F32"}


def _write_safetensors(tensors: dict[str, torch.Tensor], path: Path) -> None:
    """One safetensors file: u64 header length, JSON header, then the tensors' bytes in header order.

    Written directly (not through ``safetensors.torch.save_file``) so that several names may
    carry the same in-memory tensor: each still gets its own region of the file.
    """
    import json
    import struct

    header: dict[str, dict] = {}
    cursor = 0
    for name, t in tensors.items():
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _SAFETENSORS_DTYPES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [cursor, cursor + nbytes]}
        cursor += nbytes
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * (-len(raw) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(raw)))
        fh.write(raw)
        for t in tensors.values():
            fh.write(memoryview(t.contiguous().view(torch.uint8).numpy()))


def write_sharded_safetensors(model: nn.Module, out_dir: str | Path, blocks_per_shard: int = 4, seed: int = 0,
                              std: float = 0.02, dtype: torch.dtype = torch.bfloat16,
                              share_values: bool = True) -> dict[str, int]:
    """Frozen (``requires_grad == False``) 2-D parameters of *model* as a sharded safetensors checkpoint.

    Values are ``randn * std``.  With *share_values* the blocks all get the value set of one block
    (tensors of one shape share one draw), which keeps set-up short; every tensor still has its own
    region in the files.  Writes ``model.safetensors.index.json`` with the ``weight_map`` the sharded
    conversion reads (reference ``src/stagehand/registry.py:560-702``).  Returns ``{"tensors", "bytes", "shards"}``.
    """
    import json

    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    g = torch.Generator().manual_seed(seed)
    by_shape: dict[tuple[int, ...], torch.Tensor] = {}

    def value(shape: tuple[int, ...]) -> torch.Tensor:
        if share_values and shape in by_shape:
            return by_shape[shape]
        t = (torch.randn(shape, generator=g) * std).to(dtype)
        by_shape[shape] = t
        return t

    groups: dict[str, list[tuple[str, tuple[int, ...]]]] = {}
    for name, param in model.named_parameters():
        if param.requires_grad or param.dim() < 2:
            continue
        m = re.match(r"^(.*?\.\d+)\.", name)
        groups.setdefault(m.group(1) if m else "", []).append((name, tuple(param.shape)))
    keys = list(groups)
    weight_map: dict[str, str] = {}
    total = tensors = 0
    n_shards = (len(keys) + blocks_per_shard - 1) // blocks_per_shard
    for shard in range(n_shards):
        fname = f"model-{shard + 1:05d}-of-{n_shards:05d}.safetensors"
        payload = {}
        for key in keys[shard * blocks_per_shard:(shard + 1) * blocks_per_shard]:
            for name, shape in groups[key]:
                payload[name] = value(shape)
                weight_map[name] = fname
                total += payload[name].numel() * payload[name].element_size()
                tensors += 1
        _write_safetensors(payload, out_dir / fname)
    (out_dir / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    return {"tensors": tensors, "bytes": total, "shards": n_shards}


class EncoderPlusDiT(nn.Module):
    """A text encoder feeding a DiT: the multi-GPU sharded-streaming configuration.

    ``encoder`` is a :class:`MistralShapedEncoder`, ``dit`` a :class:`FluxShapedDiT`.  The
    encoder's output is cut to the DiT's width and used as its text stream (the real pipelines
    put a small projection there; it is not a streamed block and is left out).
    """

    def __init__(self, encoder: nn.Module, dit: nn.Module) -> None:
        super().__init__()
        self.encoder = encoder
        self.dit = dit

    def forward(self, img: torch.Tensor, text: torch.Tensor, vec: torch.Tensor) -> torch.Tensor:
        encoded = self.encoder(text)
        return self.dit(img, encoded[..., : self.dit.hidden].contiguous(), vec)


BLOCK_PATTERNS = {
    "encoder_dit": r"^(encoder\.layers|dit\.double_blocks|dit\.single_blocks)\.\d+$",
    "tiny": r"^blocks\.\d+$",
    "flux": r"^(double_blocks|single_blocks)\.\d+$",
    "mistral": r"^layers\.\d+$",
    "video": r"^blocks\.\d+$",
}


# ── synthetic SquareQ slabs ──────────────────────────────────────────────


def synth_squareq_layer(out_features: int, in_features: int, generator: torch.Generator,
                        padded_in: int | None = None, has_bias: bool = True,
                        zero_point_nonzero: bool = False, scale_median: float = 0.01) -> dict[str, torch.Tensor]:
    """One layer dict ``{qweight, scale, zero_point, bias}`` with the synthetic value distributions.

    *scale_median* is the median of the lognormal row scales (0.01 in the named configurations; a model whose
    projections have no compensating gain uses a smaller one so that activations stay finite in bf16).
    """
    padded = int(padded_in) if padded_in is not None else in_features
    q = torch.randint(-127, 128, (out_features, padded), dtype=torch.int8, generator=generator)
    scale = torch.exp(torch.randn(out_features, generator=generator) * 0.5 + math.log(scale_median)).float()
    if zero_point_nonzero:
        zp = torch.randint(-8, 9, (out_features,), generator=generator).float() * 0.5
    else:
        zp = torch.zeros(out_features, dtype=torch.float32)
    layer = {"qweight": q, "scale": scale, "zero_point": zp}
    if has_bias:
        layer["bias"] = (torch.randn(out_features, generator=generator) * 0.02).float()
    return layer


def write_squareq_fpk(model: nn.Module, block_pattern: str, path: str | Path, seed: int = 0,
                      share_storage: bool = False, pad_in_to: int | None = None,
                      scale_median: float = 0.01, distinct_scales: bool = False) -> dict[str, int]:
    """Write a SquareQ BP8 ``.fpk`` covering every ``nn.Linear`` inside the matched blocks.

    Layer names are ``"<block_id>.<linear path>"``.  With *share_storage* every
    layer of one ``(out, in)`` shape reuses a single set of tensors, so the file
    holds one copy per distinct shape (``torch.save`` writes a shared storage
    once) while the runtime still stages every block separately; this keeps the
    set-up of multi-gigabyte configurations short.  With *distinct_scales* a layer that
    shares its tensors still gets a scale vector of its own (the shared one times a
    layer-specific factor in [1, 1.06)): the file stays small, yet no two blocks expand to
    the same bytes, so a digest of a delivered block also proves that it was built from
    *its* rows and scales.  With *pad_in_to* the stored
    rows are padded to a multiple of that many columns (``padded_in > in``).

    Returns ``{"layers": n, "elements": total int8 weights}``.
    """
    generator = torch.Generator().manual_seed(seed)
    compiled = re.compile(block_pattern)
    manifest_layers: list[dict[str, object]] = []
    layers: dict[str, dict[str, torch.Tensor]] = {}
    by_shape: dict[tuple[int, int, bool], dict[str, torch.Tensor]] = {}
    elements = 0
    for block_id, block in model.named_modules():
        if not block_id or not compiled.search(block_id):
            continue
        for sub_name, sub in block.named_modules():
            if not isinstance(sub, nn.Linear):
                continue
            out_f, in_f = int(sub.out_features), int(sub.in_features)
            padded = in_f if not pad_in_to else ((in_f + pad_in_to - 1) // pad_in_to) * pad_in_to
            has_bias = sub.bias is not None
            key = (out_f, in_f, has_bias)
            if share_storage and key in by_shape:
                layer = by_shape[key]
            else:
                layer = synth_squareq_layer(out_f, in_f, generator, padded_in=padded, has_bias=has_bias,
                                            scale_median=scale_median)
                by_shape[key] = layer
            name = f"{block_id}.{sub_name}" if sub_name else block_id
            layers[name] = dict(layer)
            if distinct_scales and share_storage:
                layers[name]["scale"] = layer["scale"] * (1.0 + (len(manifest_layers) % 61) / 1024.0)
            manifest_layers.append(
                {"name": name, "out": out_f, "inp": in_f, "padded_in": padded, "has_bias": has_bias})
            elements += out_f * in_f
    payload = {
        "manifest": {
            "model_name": "synthetic",
            "quant_version": "synthetic",
            "layout": "rowwise_sym_int8",
            "pack_k": 1,
            "layers": manifest_layers,
        },
        "layers": layers,
    }
    torch.save(payload, str(path))
    return {"layers": len(manifest_layers), "elements": elements}


def materialize_small_params(model: nn.Module) -> None:
    """Give real CPU storage to the parameters of a meta-device model that no slab will ever fill.

    Large synthetic models are built on the ``meta`` device so that their projections
    (filled from the SquareQ slab at load time) never occupy host memory; the small
    module-owned parameters -- normalisation weights and biases -- need actual values:
    weights become ones, biases zeros.
    """
    for module in model.modules():
        if isinstance(module, nn.Linear):
            continue
        for name, param in list(module.named_parameters(recurse=False)):
            if param.device.type != "meta":
                continue
            fill = torch.zeros if name.endswith("bias") else torch.ones
            setattr(module, name, nn.Parameter(fill(param.shape, dtype=param.dtype), requires_grad=False))
