"""Host-side pieces of the Genesun path that need no GPU: the configuration reader, the bf16 rounding of the loader, the
safetensors reader and the sampler."""
from __future__ import annotations

import json
import struct

import numpy as np

import genesun_ref as R
from koboldcpp_b200 import genesun as G
from koboldcpp_b200.engine import Sampler


def test_layer_params_from_config():
    a = G.layer_params(R.attn_layer(heads=3, dim=24, rot_dim=12, vdim=40, kv_rank=48, q_rank=20, ff=72, rot_dims=8, kv_from=2))
    assert (a.mixer, a.heads, a.dim, a.vdim, a.rot_dim, a.kv_rank, a.q_rank, a.kv_from, a.rope_dims, a.mlp, a.ff) == (G.MIXER_LATENT_ATTENTION, 3, 24, 40, 12, 48, 20, 2, 8, G.MLP_DENSE_POLYNORM, 72)
    assert abs(a.yarn_factor - 4.0) < 1e-6 and a.yarn_original == 64
    b = G.layer_params(R.mlstm_layer(heads=2, dim=16, vdim=24, gate_cap=10.0))
    assert (b.mixer, b.heads, b.dim, b.vdim, b.kv_from, b.mlp, b.ff) == (G.MIXER_MLSTM, 2, 16, 24, -1, G.MLP_NONE, 0) and b.gate_cap == 10.0
    c = G.layer_params(R.attn_layer(scaling=False))
    assert c.yarn_factor == 0.0 and c.kv_from == -1


def test_bf16_rounding_is_to_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -3.1415927, 65504.0, 1e-30], dtype=np.float32)
    bits = G.f32_to_bf16_bits(x)
    back = (bits.astype(np.uint32) << 16).view(np.float32)
    assert np.allclose(back, R.bf16_round(x), rtol=0, atol=0)
    assert back[1] == 1.0 and back[2] == np.float32(1.015625)  # ties go to the even mantissa


def test_safetensors_reader(tmp_path):
    a = np.arange(6, dtype=np.float32).reshape(2, 3)
    b = G.f32_to_bf16_bits(np.array([0.5, -2.0], dtype=np.float32))
    head = json.dumps({"__metadata__": {}, "a": {"dtype": "F32", "shape": [2, 3], "data_offsets": [0, 24]},
                       "b": {"dtype": "BF16", "shape": [2], "data_offsets": [24, 28]}}).encode()
    (tmp_path / "m.safetensors").write_bytes(struct.pack("<Q", len(head)) + head + a.tobytes() + b.tobytes())
    t = G.read_safetensors(tmp_path / "m.safetensors")
    assert set(t) == {"a", "b"} and t["a"][1] == (2, 3)
    assert np.array_equal(G.to_f32(*t["a"][::2]).reshape(2, 3), a) and np.array_equal(G.to_f32(t["b"][0], t["b"][2]), [0.5, -2.0])


def test_sampler():
    lg = np.array([0.1, 3.0, 3.0, -1.0], dtype=np.float32)
    assert Sampler().pick(lg) == 1  # greedy: the lowest index among equals
    s = Sampler(temperature=1.0, top_k=2, seed=1)
    assert {s.pick(lg) for _ in range(50)} == {1, 2}
    assert Sampler(temperature=0.5, top_p=0.01, seed=2).pick(lg) in (1, 2)
