"""Typed configuration of the Llama 2/3 dense decoder, read from config.json's own keys.

KuiperLLama reads seven integers from its checkpoint header
(kuiper/include/model/config.h:4-15, kuiper/source/model/model.cpp:113-141) and fixes
eps, theta and the rope pairing by build flags (rmsnorm_kernel.cu:120-124,
rope_kernel.cu:4,42,128).  Here every one of them is a field read from config.json (the keys
of tools/config.json:1-26 and tools/export_llama3.py:544-554).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from .registry import ConfigError, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, default_schedule


@dataclass(frozen=True)
class Llama3RopeScaling:
    """``rope_scaling`` with ``rope_type: "llama3"``."""
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    def to_dict(self) -> dict:
        d = asdict(self)
        d["rope_type"] = "llama3"
        return d


_REQUIRED = ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
             "vocab_size", "max_position_embeddings")


@register_architecture("LlamaForCausalLM")
@dataclass(frozen=True)
class LlamaConfig:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[Llama3RopeScaling]
    tie_word_embeddings: bool
    hidden_act: str = "silu"
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    torch_dtype: str = "bfloat16"

    architecture = "LlamaForCausalLM"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LlamaConfig":
        problems: List[str] = []

        def integer(key: str, default: Any = None, required: bool = False) -> Any:
            v = d.get(key, default)
            if v is None:
                if required:
                    problems.append(f'missing key "{key}"')
                return default
            if isinstance(v, bool) or not isinstance(v, int):
                problems.append(f'"{key}" must be an integer, got {v!r}')
                return default
            if v <= 0:
                problems.append(f'"{key}" must be positive, got {v}')
            return v

        def number(key: str, default: float) -> float:
            v = d.get(key, default)
            if v is None:
                return default
            if isinstance(v, bool) or not isinstance(v, (int, float)):
                problems.append(f'"{key}" must be a number, got {v!r}')
                return default
            return float(v)

        vals = {k: integer(k, required=True) for k in _REQUIRED}
        heads = vals["num_attention_heads"]
        hidden = vals["hidden_size"]
        # kv heads default to the head count (tools/export_llama3.py:499, tools/model.py:97)
        kv_heads = integer("num_key_value_heads", heads)
        # head size = dim / heads unless config.json says otherwise (kuiper/source/model/model.cpp:123)
        head_dim = integer("head_dim", None)
        if head_dim is None and heads and hidden:
            if hidden % heads:
                problems.append(f'"hidden_size" {hidden} is not a multiple of "num_attention_heads" {heads} '
                                'and no "head_dim" is given')
            head_dim = hidden // heads
        if heads and kv_heads and heads % kv_heads:
            problems.append(f'"num_attention_heads" {heads} is not a multiple of "num_key_value_heads" {kv_heads}')
        if head_dim is not None and head_dim % 2:
            problems.append(f'"head_dim" {head_dim} must be even for rotary pairs')

        # eps: 1e-5 is what KuiperLLama's Llama build compiles in (rmsnorm_kernel.cu:123);
        # theta: 10000 is its default build (rope_kernel.cu:128).
        eps = number("rms_norm_eps", 1e-5)
        theta = number("rope_theta", 10000.0)
        if eps <= 0:
            problems.append(f'"rms_norm_eps" must be positive, got {eps}')
        if theta <= 0:
            problems.append(f'"rope_theta" must be positive, got {theta}')

        scaling = None
        rs = d.get("rope_scaling")
        if rs is not None:
            if not isinstance(rs, dict):
                problems.append(f'"rope_scaling" must be null or an object, got {rs!r}')
            else:
                kind = rs.get("rope_type", rs.get("type"))
                if kind in (None, "default"):
                    scaling = None
                elif kind != "llama3":
                    problems.append(f'unsupported rope_scaling type {kind!r} (supported: "llama3", "default", null)')
                else:
                    missing = [k for k in ("factor", "low_freq_factor", "high_freq_factor",
                                           "original_max_position_embeddings") if k not in rs]
                    if missing:
                        problems.append(f'"rope_scaling" lacks {missing}')
                    else:
                        scaling = Llama3RopeScaling(float(rs["factor"]), float(rs["low_freq_factor"]),
                                                    float(rs["high_freq_factor"]),
                                                    int(rs["original_max_position_embeddings"]))
                        if scaling.high_freq_factor <= scaling.low_freq_factor:
                            problems.append('"rope_scaling": high_freq_factor must exceed low_freq_factor')
                        if scaling.factor <= 0:
                            problems.append('"rope_scaling": factor must be positive')

        act = d.get("hidden_act", "silu")
        if act != "silu":   # the only activation KuiperLLama has (swiglu_kernel.cu:18-21)
            problems.append(f'unsupported "hidden_act" {act!r} (supported: "silu")')
        for key in ("attention_bias", "mlp_bias"):   # no bias anywhere (tools/model.py:104-107,174-176)
            if d.get(key, False):
                problems.append(f'"{key}": true is not supported (this decoder has no biases)')

        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = tuple(eos)
        else:
            problems.append(f'"eos_token_id" must be an integer or a list of integers, got {eos!r}')
            eos_ids = ()
        bos = d.get("bos_token_id")
        if bos is not None and (isinstance(bos, bool) or not isinstance(bos, int)):
            problems.append(f'"bos_token_id" must be an integer, got {bos!r}')
            bos = None

        if problems:
            raise ConfigError("config.json (LlamaForCausalLM): " + "; ".join(problems))
        return cls(hidden_size=hidden, intermediate_size=vals["intermediate_size"],
                   num_hidden_layers=vals["num_hidden_layers"], num_attention_heads=heads,
                   num_key_value_heads=kv_heads, head_dim=head_dim, vocab_size=vals["vocab_size"],
                   max_position_embeddings=vals["max_position_embeddings"], rms_norm_eps=eps,
                   rope_theta=theta, rope_scaling=scaling,
                   tie_word_embeddings=bool(d.get("tie_word_embeddings", False)), hidden_act=act,
                   bos_token_id=bos, eos_token_ids=eos_ids,
                   torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))))

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        d = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None if self.rope_scaling is None else self.rope_scaling.to_dict(),
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "attention_bias": False,
            "mlp_bias": False,
            "torch_dtype": self.torch_dtype,
        }
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        return d

    # ------------------------------------------------------------------ the model it describes
    def to_model_spec(self) -> ModelSpec:
        """Pre-norm residual blocks of (RMSNorm, rotary GQA attention, RMSNorm, SwiGLU)
        in layer order (kuiper/source/model/llama3.cpp:155-164)."""
        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        rope = PartSpec("rope", {
            "head_dim": self.head_dim, "theta": self.rope_theta,
            "scaling": None if self.rope_scaling is None else self.rope_scaling.to_dict(),
        })
        mixer = PartSpec("attention", {
            "hidden_size": self.hidden_size, "num_heads": self.num_attention_heads,
            "num_kv_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "window": None,
            "names": {"q": "self_attn.q_proj.weight", "k": "self_attn.k_proj.weight",
                      "v": "self_attn.v_proj.weight", "o": "self_attn.o_proj.weight"},
        })
        ffn = PartSpec("swiglu", {
            "hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size,
            "names": {"gate": "mlp.gate_proj.weight", "up": "mlp.up_proj.weight",
                      "down": "mlp.down_proj.weight"},
        })
        layers = tuple(
            LayerSpec(prefix=f"model.layers.{i}.", arrangement="pre_norm", mixer=mixer, feed_forward=ffn,
                      mixer_norm=PartSpec("rmsnorm", {**norm.params, "name": "input_layernorm.weight"}),
                      feed_forward_norm=PartSpec("rmsnorm", {**norm.params, "name": "post_attention_layernorm.weight"}),
                      position=rope)
            for i in range(self.num_hidden_layers))
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=self.hidden_size, vocab_size=self.vocab_size,
            max_positions=self.max_position_embeddings, layers=layers,
            schedule=default_schedule(self.num_hidden_layers),
            embedding_name="model.embed_tokens.weight",
            final_norm=PartSpec("rmsnorm", {**norm.params, "name": "weight"}), final_norm_prefix="model.norm.",
            lm_head_name=None if self.tie_word_embeddings else "lm_head.weight",
            stop_token_ids=self.eos_token_ids, bos_token_id=self.bos_token_id,
            # exporters of Llama checkpoints may write rotary tables, and a classifier beside a tied table
            ignorable_suffixes=("rotary_emb.inv_freq",) + (("lm_head.weight",) if self.tie_word_embeddings else ()))
        spec.validate()
        return spec
