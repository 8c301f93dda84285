"""Typed LFM2 configuration, read from the architecture's own config.json keys.

LFM2 is a stack of pre-norm blocks whose mixer is either a double-gated short
convolution or grouped-query attention with per-head q/k RMSNorm and RoPE,
each followed by a SwiGLU feed-forward.  The reference reads the same facts
from GGUF metadata (src/Inference/lfm2.jl:32-152): per-layer KV head counts
with 0 meaning "conv layer" (:50-58, :114), ``shortconv.l_cache`` (:114),
``rope.freq_base`` (:146), ``attention.layer_norm_rms_epsilon`` (:151), and it
refuses every key it does not know (:43-47).  The config.json spellings below
are this engine's; the refusal policy is the reference's.

Feed-forward width: ``block_ff_dim`` is the nominal width.  With
``block_auto_adjust_ff_dim`` it becomes ``floor(2*ff/3)``, then
``floor(block_ffn_dim_multiplier * ff)`` when a multiplier is given, then it is
rounded up to a multiple of ``block_multiple_of``
(12288 -> 8192 at 256; 6656 -> 4608; 10240 -> 6912; 384 -> 256 at 32).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..errors import invalid
from .registry import register_architecture
from .spec import BlockSpec, ModelSpec, PartSpec, default_schedule

ARCHITECTURE = "Lfm2ForCausalLM"
MODEL_TYPE = "lfm2"

# Keys that describe the architecture.
_KEYS = {
    "architectures", "model_type", "vocab_size", "hidden_size", "num_hidden_layers",
    "num_attention_heads", "num_key_value_heads", "head_dim", "layer_types", "full_attn_idxs",
    "conv_L_cache", "conv_bias", "block_ff_dim", "block_auto_adjust_ff_dim",
    "block_multiple_of", "block_ffn_dim_multiplier", "intermediate_size", "norm_eps",
    "rope_theta", "tie_embedding", "tie_word_embeddings", "max_position_embeddings",
    "bos_token_id", "eos_token_id", "pad_token_id",
}
# Bookkeeping keys of checkpoint folders that change nothing the engine computes.
_IGNORED_KEYS = {
    "transformers_version", "torch_dtype", "dtype", "use_cache", "initializer_range",
    "_name_or_path", "use_pos_enc", "block_dim", "block_mlp_init_scale", "block_out_init_scale",
    "block_use_swiglu", "block_use_xavier_init", "conv_dim", "conv_dim_out",
    "conv_use_xavier_init", "block_norm_eps",
}

_LAYER_KINDS = {"conv": False, "full_attention": True}


def effective_ff_dim(block_ff_dim: int, auto_adjust: bool, multiple_of: int,
                     multiplier: Optional[float]) -> int:
    ff = int(block_ff_dim)
    if auto_adjust:
        ff = (2 * ff) // 3
        if multiplier is not None:
            ff = int(float(multiplier) * ff)
        ff = multiple_of * ((ff + multiple_of - 1) // multiple_of)
    return ff


@dataclass(frozen=True)
class Lfm2Config:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    layer_is_attention: Tuple[bool, ...]
    conv_L_cache: int
    conv_bias: bool
    ff_dim: int                      # effective feed-forward width
    norm_eps: float
    rope_theta: float
    tie_embedding: bool
    max_position_embeddings: Optional[int] = None
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    pad_token_id: Optional[int] = None

    # ---- parsing -------------------------------------------------------------------
    @staticmethod
    def from_json(cfg: Mapping[str, Any]) -> "Lfm2Config":
        for k in cfg:
            if k not in _KEYS and k not in _IGNORED_KEYS:
                raise invalid(f"LFM2 config: unsupported key {k!r} (no LFM2 feature declares it)")

        def req_int(key: str, minimum: int = 1) -> int:
            if key not in cfg:
                raise invalid(f"LFM2 config: missing {key!r}")
            v = cfg[key]
            if isinstance(v, bool) or not isinstance(v, int):
                raise invalid(f"LFM2 config: {key!r} must be an integer, got {v!r}")
            if v < minimum:
                raise invalid(f"LFM2 config: {key!r} must be >= {minimum}, got {v}")
            return v

        def opt_int(key: str) -> Optional[int]:
            v = cfg.get(key)
            if v is None:
                return None
            if isinstance(v, bool) or not isinstance(v, int):
                raise invalid(f"LFM2 config: {key!r} must be an integer, got {v!r}")
            return v

        def opt_bool(key: str, default: bool) -> bool:
            v = cfg.get(key, default)
            if not isinstance(v, bool):
                raise invalid(f"LFM2 config: {key!r} must be true or false, got {v!r}")
            return v

        def opt_float(key: str, default: float) -> float:
            v = cfg.get(key, default)
            if isinstance(v, bool) or not isinstance(v, (int, float)):
                raise invalid(f"LFM2 config: {key!r} must be a number, got {v!r}")
            return float(v)

        vocab = req_int("vocab_size")
        hidden = req_int("hidden_size")
        n_layers = req_int("num_hidden_layers")
        n_heads = req_int("num_attention_heads")
        n_kv = req_int("num_key_value_heads")
        if hidden % n_heads != 0:
            raise invalid(f"LFM2 config: hidden_size {hidden} is not a multiple of num_attention_heads {n_heads}")
        head_dim = opt_int("head_dim") or hidden // n_heads
        # the attention width must equal the hidden width (src/Inference/lfm2.jl:63-65)
        if n_heads * head_dim != hidden:
            raise invalid(
                f"LFM2 config: num_attention_heads*head_dim = {n_heads * head_dim} must equal hidden_size {hidden}")
        if head_dim % 2 != 0:
            raise invalid(f"LFM2 config: head_dim {head_dim} must be even (rotary pairs)")
        if n_heads % n_kv != 0:
            raise invalid(f"LFM2 config: num_attention_heads {n_heads} is not a multiple of num_key_value_heads {n_kv}")

        # layer pattern: layer_types or full_attn_idxs; both must agree when both are given
        by_types = None
        if "layer_types" in cfg:
            lt = cfg["layer_types"]
            if not isinstance(lt, list) or len(lt) != n_layers:
                raise invalid(f"LFM2 config: 'layer_types' must list {n_layers} layers")
            for i, v in enumerate(lt):
                if v not in _LAYER_KINDS:
                    raise invalid(f"LFM2 config: layer_types[{i}] = {v!r}; known kinds: {sorted(_LAYER_KINDS)}")
            by_types = tuple(_LAYER_KINDS[v] for v in lt)
        by_idxs = None
        if "full_attn_idxs" in cfg:
            idxs = cfg["full_attn_idxs"]
            if not isinstance(idxs, list) or any(isinstance(i, bool) or not isinstance(i, int) for i in idxs):
                raise invalid("LFM2 config: 'full_attn_idxs' must be a list of layer indices")
            if sorted(set(idxs)) != idxs:
                raise invalid("LFM2 config: 'full_attn_idxs' must be sorted and without repeats")
            if idxs and (idxs[0] < 0 or idxs[-1] >= n_layers):
                raise invalid(f"LFM2 config: 'full_attn_idxs' has an index outside 0..{n_layers - 1}")
            by_idxs = tuple(i in set(idxs) for i in range(n_layers))
        if by_types is None and by_idxs is None:
            raise invalid("LFM2 config: missing 'layer_types' (or 'full_attn_idxs')")
        if by_types is not None and by_idxs is not None and by_types != by_idxs:
            raise invalid("LFM2 config: 'layer_types' and 'full_attn_idxs' disagree")
        is_attn = by_types if by_types is not None else by_idxs

        L = cfg.get("conv_L_cache", 3)
        if isinstance(L, bool) or not isinstance(L, int) or L < 2:
            # a kernel of one tap keeps no history (src/Inference/architecture_spec.jl:175)
            raise invalid(f"LFM2 config: 'conv_L_cache' must be an integer >= 2, got {L!r}")
        conv_bias = opt_bool("conv_bias", False)

        auto = opt_bool("block_auto_adjust_ff_dim", False)
        multiple_of = cfg.get("block_multiple_of", 256)
        if isinstance(multiple_of, bool) or not isinstance(multiple_of, int) or multiple_of < 1:
            raise invalid(f"LFM2 config: 'block_multiple_of' must be a positive integer, got {multiple_of!r}")
        mult = cfg.get("block_ffn_dim_multiplier")
        if mult is not None and (isinstance(mult, bool) or not isinstance(mult, (int, float)) or mult <= 0):
            raise invalid(f"LFM2 config: 'block_ffn_dim_multiplier' must be a positive number, got {mult!r}")
        inter = opt_int("intermediate_size")
        if "block_ff_dim" in cfg:
            ff = effective_ff_dim(req_int("block_ff_dim"), auto, multiple_of, mult)
            if inter is not None and inter != ff:
                raise invalid(
                    f"LFM2 config: 'intermediate_size' {inter} differs from the width {ff} that 'block_ff_dim' gives")
        elif inter is not None:
            if inter < 1:
                raise invalid("LFM2 config: 'intermediate_size' must be positive")
            ff = inter
        else:
            raise invalid("LFM2 config: missing 'block_ff_dim' (or 'intermediate_size')")

        eps = opt_float("norm_eps", 1e-5)
        if not eps > 0:
            raise invalid(f"LFM2 config: 'norm_eps' must be > 0, got {eps}")
        theta = opt_float("rope_theta", 1e6)
        if not theta > 0:
            raise invalid(f"LFM2 config: 'rope_theta' must be > 0, got {theta}")
        if "tie_embedding" in cfg and "tie_word_embeddings" in cfg and \
                cfg["tie_embedding"] != cfg["tie_word_embeddings"]:
            raise invalid("LFM2 config: 'tie_embedding' and 'tie_word_embeddings' disagree")
        tie = opt_bool("tie_embedding", opt_bool("tie_word_embeddings", True))

        return Lfm2Config(
            vocab_size=vocab, hidden_size=hidden, num_hidden_layers=n_layers,
            num_attention_heads=n_heads, num_key_value_heads=n_kv, head_dim=head_dim,
            layer_is_attention=is_attn, conv_L_cache=L, conv_bias=conv_bias, ff_dim=ff,
            norm_eps=eps, rope_theta=theta, tie_embedding=tie,
            max_position_embeddings=opt_int("max_position_embeddings"),
            bos_token_id=opt_int("bos_token_id"), eos_token_id=opt_int("eos_token_id"),
            pad_token_id=opt_int("pad_token_id"),
        )

    # ---- the config.json this configuration is written as ------------------------------
    def to_json(self) -> dict:
        out = {
            "architectures": [ARCHITECTURE], "model_type": MODEL_TYPE,
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "layer_types": ["full_attention" if a else "conv" for a in self.layer_is_attention],
            "conv_L_cache": self.conv_L_cache, "conv_bias": self.conv_bias,
            "block_ff_dim": self.ff_dim, "block_auto_adjust_ff_dim": False,
            "norm_eps": self.norm_eps, "rope_theta": self.rope_theta,
            "tie_embedding": self.tie_embedding,
        }
        for k in ("max_position_embeddings", "bos_token_id", "eos_token_id", "pad_token_id"):
            v = getattr(self, k)
            if v is not None:
                out[k] = v
        return out

    # ---- the model this configuration describes ---------------------------------------
    def to_spec(self) -> ModelSpec:
        H = self.hidden_size
        norm = PartSpec("rmsnorm", {"size": H, "eps": self.norm_eps})
        ff = PartSpec("swiglu", {"hidden_size": H, "ff_dim": self.ff_dim})
        attention = PartSpec("gqa_attention", {
            "hidden_size": H, "n_heads": self.num_attention_heads,
            "n_kv_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "qk_norm_eps": self.norm_eps, "window": None,
            "position": PartSpec("rope", {"theta": self.rope_theta, "rotary_dim": self.head_dim}),
        })
        conv = PartSpec("short_conv", {"hidden_size": H, "kernel": self.conv_L_cache,
                                       "bias": self.conv_bias})
        blocks = []
        names = {
            "embedding.weight": ("model.embed_tokens.weight", "token_embd.weight"),
            # the tensor called "embedding norm" is the norm before the output head
            # (src/Inference/lfm2.jl:106-110, 173)
            "final_norm.weight": ("model.embedding_norm.weight", "token_embd_norm.weight"),
            "lm_head.weight": ("lm_head.weight", "output.weight"),
        }
        for i, is_attn in enumerate(self.layer_is_attention):
            p = f"layers.{i}."
            hf, gg = f"model.layers.{i}.", f"blk.{i}."
            blocks.append(BlockSpec("prenorm", attention if is_attn else conv, ff, norm, norm, p))
            names[p + "mixer_norm.weight"] = (hf + "operator_norm.weight", gg + "attn_norm.weight")
            names[p + "ff_norm.weight"] = (hf + "ffn_norm.weight", gg + "ffn_norm.weight")
            # GGUF-style names as the reference lists them (src/Inference/lfm2.jl:156-176)
            names[p + "feed_forward.gate_proj.weight"] = (hf + "feed_forward.w1.weight", gg + "ffn_gate.weight")
            names[p + "feed_forward.up_proj.weight"] = (hf + "feed_forward.w3.weight", gg + "ffn_up.weight")
            names[p + "feed_forward.down_proj.weight"] = (hf + "feed_forward.w2.weight", gg + "ffn_down.weight")
            if is_attn:
                for ours, h_name, g_name in (
                        ("q_proj", "self_attn.q_proj", "attn_q"), ("k_proj", "self_attn.k_proj", "attn_k"),
                        ("v_proj", "self_attn.v_proj", "attn_v"), ("o_proj", "self_attn.out_proj", "attn_output"),
                        ("q_norm", "self_attn.q_layernorm", "attn_q_norm"),
                        ("k_norm", "self_attn.k_layernorm", "attn_k_norm")):
                    names[p + f"mixer.{ours}.weight"] = (hf + h_name + ".weight", gg + g_name + ".weight")
            else:
                for ours, g_name in (("in_proj", "shortconv.in_proj"), ("conv", "shortconv.conv"),
                                     ("out_proj", "shortconv.out_proj")):
                    names[p + f"mixer.{ours}.weight"] = (hf + f"conv.{ours}.weight", gg + g_name + ".weight")
                    if self.conv_bias:
                        names[p + f"mixer.{ours}.bias"] = (hf + f"conv.{ours}.bias", gg + g_name + ".bias")
        return ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab_size, hidden_size=H,
            blocks=tuple(blocks), schedule=default_schedule(len(blocks)), final_norm=norm,
            tie_embedding=self.tie_embedding, tensor_names=names,
            ignorable_tensors=(r".*rotary_emb\.inv_freq$",),
            bos_token_id=self.bos_token_id, eos_token_id=self.eos_token_id,
            max_position=self.max_position_embeddings, source=self,
        )


def lfm2_adapter(cfg: Mapping[str, Any]) -> ModelSpec:
    return Lfm2Config.from_json(cfg).to_spec()


lfm2_adapter.model_type = MODEL_TYPE
register_architecture(ARCHITECTURE, lfm2_adapter, replace=True)
