"""Node list of the LUT engine's model graph for the Llama/Qwen2 family.

Mirrors ``UnifiedConfig::from_file`` (src/lut/graph.rs:217-292) and
``ModelGraph::build`` (src/lut/graph.rs:304-531) for the standard
full-attention layer: per layer Norm, Q, K, V, RoPE, SDPA, O, Norm, Gate, Up,
Activation, Down; then the final Norm and, when embeddings are untied, the LM
head.  The engine's device step is compiled from exactly this order.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import List, Tuple


@dataclass
class UnifiedConfig:
    vocab_size: int = 151936
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 32
    head_dim: int = 128
    norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    activation: str = "silu"
    tie_word_embeddings: bool = False
    key_prefix: str = "model"

    @classmethod
    def from_file(cls, path: str) -> "UnifiedConfig":
        with open(path) as f:
            raw = json.load(f)
        return cls.from_dict(raw)

    @classmethod
    def from_dict(cls, raw: dict) -> "UnifiedConfig":
        def get(name, default=None):
            # cascading resolution: text_config > language_config > root (graph.rs resolve_cfg!)
            for blk in (raw.get("text_config"), raw.get("language_config"), raw):
                if isinstance(blk, dict) and blk.get(name) is not None:
                    return blk[name]
            return default

        hidden = get("hidden_size", 4096)
        heads = get("num_attention_heads", 32)
        theta = None
        for blk in (raw.get("text_config"), raw.get("language_config"), raw):
            if isinstance(blk, dict):
                rp = blk.get("rope_parameters")
                if isinstance(rp, dict) and rp.get("rope_theta") is not None:
                    theta = rp["rope_theta"]
                    break
                if blk.get("rope_theta") is not None:
                    theta = blk["rope_theta"]
                    break
        act = get("hidden_act")
        return cls(
            vocab_size=get("vocab_size", 151936), hidden_size=hidden,
            intermediate_size=get("intermediate_size", 11008), num_layers=get("num_hidden_layers", 32),
            num_heads=heads, num_kv_heads=get("num_key_value_heads", heads),
            head_dim=get("head_dim", hidden // heads),
            norm_eps=get("rms_norm_eps", get("layer_norm_eps", 1e-5)),
            rope_theta=float(theta) if theta is not None else 10000.0,
            activation="gelu" if act in ("gelu", "gelu_pytorch_tanh") else "silu",
            tie_word_embeddings=bool(get("tie_word_embeddings", False)))


@dataclass
class ModelGraph:
    nodes: List[Tuple] = field(default_factory=list)
    num_layers: int = 0

    @classmethod
    def build(cls, c: UnifiedConfig) -> "ModelGraph":
        p = c.key_prefix
        nodes: List[Tuple] = [("TokenEmbedding", f"{p}.embed_tokens.weight", c.vocab_size, c.hidden_size)]
        q_dim, kv_dim = c.num_heads * c.head_dim, c.num_kv_heads * c.head_dim
        for i in range(c.num_layers):
            pre = f"{p}.layers.{i}"
            nodes += [
                ("Norm", f"{pre}.input_layernorm.weight", c.norm_eps),
                ("PalettizedMatmul", "q", f"{pre}.self_attn.q_proj.weight", q_dim, c.hidden_size),
                ("PalettizedMatmul", "k", f"{pre}.self_attn.k_proj.weight", kv_dim, c.hidden_size),
                ("PalettizedMatmul", "v", f"{pre}.self_attn.v_proj.weight", kv_dim, c.hidden_size),
                ("RotaryEmbedding", c.head_dim, c.rope_theta),
                ("ScaledDotProductAttention", c.num_heads, c.num_kv_heads, c.head_dim),
                ("PalettizedMatmul", "o", f"{pre}.self_attn.o_proj.weight", c.hidden_size, q_dim),
                ("Norm", f"{pre}.post_attention_layernorm.weight", c.norm_eps),
                ("PalettizedMatmul", "gate", f"{pre}.mlp.gate_proj.weight", c.intermediate_size, c.hidden_size),
                ("PalettizedMatmul", "up", f"{pre}.mlp.up_proj.weight", c.intermediate_size, c.hidden_size),
                ("Activation", c.activation),
                ("PalettizedMatmul", "down", f"{pre}.mlp.down_proj.weight", c.hidden_size, c.intermediate_size),
            ]
        nodes.append(("Norm", f"{p}.norm.weight", c.norm_eps))
        if not c.tie_word_embeddings:
            nodes.append(("LanguageModelHead", f"{p}.lm_head.weight", c.vocab_size, c.hidden_size))
        return cls(nodes=nodes, num_layers=c.num_layers)

    def palettized_tensors(self):
        """(key, dim_m, dim_n) of every matmul tensor (graph.rs:533-544)."""
        out = []
        for n in self.nodes:
            if n[0] == "PalettizedMatmul":
                out.append((n[2], n[3], n[4]))
            elif n[0] == "LanguageModelHead":
                out.append((n[1], n[2], n[3]))
        return out

    def embedding(self):
        n = self.nodes[0]
        return n[1], n[2], n[3]


def generate_plan(graph: ModelGraph, has_gpu: bool = True) -> str:
    """``generate_plan`` (src/lut/graph.rs:592-654) serialised as serde_json writes ``ExecutionPlan``
    (:552-589): one backend assignment per node, the KV format and the attention strategy the compiler
    assumed.  ``has_gpu`` plays the role of ``has_metal``; the variant names are the reference's."""
    gemm = "MetalGemm" if has_gpu else "CpuGemm"
    per_node = {"TokenEmbedding": "Skip", "Norm": "CpuNorm", "PalettizedMatmul": gemm, "RotaryEmbedding": "CpuRope",
                "ScaledDotProductAttention": "MetalAttention" if has_gpu else "CpuSoftmaxAttn",
                "Activation": "CpuActivation", "LanguageModelHead": gemm}
    plan = {"version": 1, "architecture": "prism-engine", "num_layers": graph.num_layers,
            "node_backends": [per_node[n[0]] for n in graph.nodes],
            "kv_cache": "Fp16" if has_gpu else "Int8",
            "attention_strategy": "MetalKernel" if has_gpu else "CpuSoftmax",
            "lm_head_backend": "metal" if has_gpu else "cpu"}
    return json.dumps(plan, separators=(",", ":"))
