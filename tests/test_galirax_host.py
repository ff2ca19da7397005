"""Host-side pieces of the Galirax path that need no GPU: the configuration reader, the order of layer runs, the registry and
the reference's own consistency (rotation bands, router)."""
from __future__ import annotations

import numpy as np
import pytest

import galirax_ref as R
from koboldcpp_b200 import galirax as G
from koboldcpp_b200 import models
from koboldcpp_b200.lib import B200Error


def test_layer_params_from_config():
    a = G.layer_params(R.attn_layer("attention_2", heads=6, kv_heads=2, dim=8, vdim=4, rot_dims=2, window=4, keep_first=1, mlp=R.moe(ff=8, experts=12, top=4, groups=4, keep=2, scale=0.7)))
    assert (a.mixer, a.heads, a.kv_heads, a.dim, a.vdim, a.rope_dims, a.window, a.keep_first, a.qkv_bias, a.qk_norm) == (G.MIXER_ATTENTION, 6, 2, 8, 4, 2, 4, 1, 1, 1)
    assert (a.mlp, a.ff, a.n_expert, a.n_expert_used, a.n_group, a.n_group_used) == (G.MLP_MOE_GATED, 8, 12, 4, 4, 2) and abs(a.router_scale - 0.7) < 1e-6
    assert a.rope_scaling == G.ROPE_SCALING_BANDS and (a.yarn_factor, a.band_low, a.band_high, a.yarn_original) == (4.0, 1.0, 3.0, 48)
    b = G.layer_params(R.attn_layer(scaling=False, mlp=None))
    assert (b.qkv_bias, b.qk_norm, b.window, b.rope_scaling, b.mlp) == (0, 0, 0, G.ROPE_SCALING_NONE, G.MLP_NONE)
    c = G.layer_params(R.lightning_layer(heads=2, dim=16, vdim=24))
    assert (c.mixer, c.heads, c.dim, c.vdim) == (G.MIXER_LIGHTNING, 2, 16, 24)
    assert G.decays({"heads": 3, "decay": 0.5}) == [0.5, 0.5, 0.5] and G.decays({"heads": 2, "decay": [0.25, 0.75]}) == [0.25, 0.75]
    with pytest.raises(B200Error):
        G.layer_params({"type": "convolution", "mixer": {}, "mlp": None})
    with pytest.raises(B200Error):
        G.layer_params(R.lightning_layer(heads=3, decay=[0.5]))


def test_run_order():
    assert G.run_order(4, None) == [0, 1, 2, 3]
    assert G.run_order(6, {"start": 1, "stop": 3, "times": 3}) == [0, 1, 2, 1, 2, 1, 2, 3, 4, 5]
    assert G.run_order(3, {"start": 0, "stop": 3, "times": 2}) == [0, 1, 2, 0, 1, 2]
    assert G.run_order(3, {"start": 2, "stop": 2, "times": 5}) == [0, 1, 2]
    with pytest.raises(B200Error):
        G.run_order(3, {"start": 2, "stop": 4, "times": 2})
    cfg = R.make_config([R.attn_layer(), R.lightning_layer()], loop=(1, 2, 3))
    assert R.run_order(cfg) == G.run_order(2, cfg["loop"])


def test_registry_knows_the_architecture():
    assert models.ARCHITECTURES["Galirax"] is G.load


def test_reference_rotation_bands_and_router():
    rot = {"base": 10000.0, "dims": 32, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}
    f, plain = R.rotation_freqs(rot), R.rotation_freqs({"base": 10000.0, "dims": 32})
    wl = 2 * np.pi / plain
    assert np.allclose(f[wl < 16], plain[wl < 16]) and np.allclose(f[wl > 64], plain[wl > 64] / 8.0)
    mid = (wl >= 16) & (wl <= 64)
    assert mid.any() and (f[mid] <= plain[mid] + 1e-15).all() and (f[mid] >= plain[mid] / 8.0 - 1e-15).all()
    # groups: expert 5 has the best score but its group loses on the sum of its two best
    z = np.array([2.0, 2.0, -9.0, -9.0, -9.0, 2.5])
    chosen, w = R.route(z, np.zeros(6), 2, 3, 1, 2.0)
    assert chosen == [0, 1] and abs(w.sum() - 2.0) < 1e-12
    chosen, _ = R.route(z, np.array([0, 0, 0, 0, 3.0, 0]), 2, 3, 1, 1.0)  # the correction moves the choice, not the weights
    assert chosen == [4, 5]
