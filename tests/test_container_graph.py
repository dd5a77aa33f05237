"""Container and graph host logic against the reference's own tests (CPU)."""
import json
import os

import numpy as np

from prism_engine_b200 import CImageReader, CImageWriter, ModelGraph, UnifiedConfig, synth

QWEN2_FIXTURE = {  # tests/fixtures/lut_graph/qwen2_config.json of the reference
    "architectures": ["Qwen2ForCausalLM"], "vocab_size": 151936, "hidden_size": 896, "intermediate_size": 4864,
    "num_hidden_layers": 24, "num_attention_heads": 14, "num_key_value_heads": 2, "head_dim": 64,
    "rms_norm_eps": 1e-6, "rope_theta": 1000000, "hidden_act": "silu", "tie_word_embeddings": True}


def test_cimage_roundtrip(tmp_path):
    # src/quantization/cimage.rs:360-390: dims preserved, offsets 16 KB aligned
    p = str(tmp_path / "t.cimage")
    w = CImageWriter(p)
    pay = synth.make_payload(64, 32, seed=3)
    w.append_palettized("model.layers.0.mlp.up_proj.weight", pay, 64, 32)
    w.append_fp16("norm", np.zeros(128, np.uint8), 1, 64)
    w.append_blob("blob", np.arange(10, dtype=np.uint8))
    w.set_execution_plan(json.dumps({"has_metal": False}))
    w.finalize()
    r = CImageReader(p)
    rec = r.tensor("model.layers.0.mlp.up_proj.weight")
    assert rec["dim_m"] == 64 and rec["dim_n"] == 32 and rec["offset"] % 16384 == 0
    assert rec["offset"] >= 8 * 16384 and rec["tensor_type"] == "Palettized4Bit"
    assert np.array_equal(r.read_payload("model.layers.0.mlp.up_proj.weight"), pay)
    assert r.tensor("blob")["offset"] % 16384 == 0 and r.tensor("missing") is None
    assert json.loads(r.execution_plan) == {"has_metal": False}
    raw = open(p, "rb").read(16)
    assert raw[:8] == b"TRB_CIMG"


def test_cimage_many_tensors(tmp_path):
    # src/quantization/cimage.rs:392-411: 50 tensors fit the reserved header
    p = str(tmp_path / "many.cimage")
    w = CImageWriter(p)
    for i in range(50):
        w.append_palettized(f"model.layers.{i}.self_attn.q_proj.weight", synth.make_payload(8, 32, seed=i), 8, 32)
    w.finalize()
    r = CImageReader(p)
    assert len(r.tensors) == 50
    assert os.path.getsize(p) >= 8 * 16384 + 49 * 16384


def test_qwen2_graph_counts():
    # src/lut/graph.rs:660-703: 1 + 24*12 + 1 nodes, 168 palettized tensors, theta 1e6, tied
    c = UnifiedConfig.from_dict(QWEN2_FIXTURE)
    g = ModelGraph.build(c)
    assert len(g.nodes) == 290 and g.num_layers == 24
    assert len(g.palettized_tensors()) == 168
    assert c.rope_theta == 1e6 and c.tie_word_embeddings and c.head_dim == 64
    assert g.nodes[0][0] == "TokenEmbedding" and g.nodes[-1][0] == "Norm"
    order = [n[0] if n[0] != "PalettizedMatmul" else n[1] for n in g.nodes[1:13]]
    assert order == ["Norm", "q", "k", "v", "RotaryEmbedding", "ScaledDotProductAttention", "o", "Norm", "gate",
                     "up", "Activation", "down"]


def test_untied_graph_has_head():
    c = UnifiedConfig.from_dict(dict(QWEN2_FIXTURE, tie_word_embeddings=False, num_hidden_layers=2))
    g = ModelGraph.build(c)
    assert g.nodes[-1][0] == "LanguageModelHead" and len(g.palettized_tensors()) == 15


def test_algorithmic_bytes():
    assert synth.gemv_algorithmic_bytes(4864, 896) == 2346240
    assert synth.payload_bytes(4864, 896) == 155648 + 2179072
