"""Kogonex without a GPU: its configuration, the model as data, what its layers ask of the cache
manager, the scaled rotary constants, and properties of the plain implementation itself."""

import math

import pytest
import torch

from acorninfer_b200.cache.manager import CacheManager
from acorninfer_b200.config.model_config import ConfigError, KogonexConfig
from acorninfer_b200.models.decoder import Decoder, expected_tensors
from acorninfer_b200.parts.base import BuildContext
from acorninfer_b200.parts.rope import ScaledRope
from acorninfer_b200.registry import config_from_dict, spec_for
from tests.kogonex_tiny import KOGOS
from tests.plain import kogonex as plain
from tests.tiny import random_tokens


@pytest.mark.parametrize("name", list(KOGOS))
def test_config_round_trip_and_registry(name):
    cfg = KOGOS[name]["cfg"]
    raw = cfg.to_dict()
    assert raw["architecture"] == "Kogonex" and len(raw["layers"]) == len(cfg.layers)
    again = config_from_dict(raw)
    assert isinstance(again, KogonexConfig) and again == cfg


def test_config_errors_name_the_key():
    raw = KOGOS["kogo_a"]["cfg"].to_dict()
    for path, value, word in ((("layers", 0, "type"), "conv_mixer", "type"), (("layers", 2, "mixer", "kv_from"), 1, "kv_from"),
                              (("layers", 0, "mlp", "router", "top"), 5, "choices"), (("norm", "eps"), 0.0, "eps")):
        import copy
        bad = copy.deepcopy(raw)
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            config_from_dict(bad)
    bad = copy.deepcopy(raw)
    del bad["layers"][1]["mixer"]["conv"]
    with pytest.raises(ConfigError, match="conv"):
        config_from_dict(bad)


def test_model_as_data_and_cache_needs():
    cfg = KOGOS["kogo_a"]["cfg"]
    spec = spec_for(cfg)
    assert [e.reads_cache_of for e in spec.schedule] == [None, None, 0, None]
    assert spec.layers[1].feed_forward is None and set(spec.layers[1].norms) == {"mixer"}
    names = expected_tensors(spec)
    for n in ("embed", "bigram", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.dkv.norm", "l0.mix.sink", "l1.mix.q.conv",
              "l1.mix.A_log", "l1.mix.dt_bias", "l2.mix.uk", "l3.mlp.e2.down", "l3.mlp.correction"):
        assert n in names, n
    assert "l2.mix.dkv" not in names and "l1.norm2" not in names and "l2.mlp.e5.gate" not in names
    assert names["bigram"].shape == (cfg.bigram_buckets + 1, cfg.hidden_size)
    dec = Decoder(spec, torch.float32, "cpu", page_size=8)
    kv, state = dec.cache_needs()
    # layer 0 keeps latent + rotated key part, one row per token, for the wider of the two windows that read it
    assert set(kv) == {0} and kv[0].head_dim == 48 and kv[0].num_kv_heads == 1 and not kv[0].values and kv[0].window == 21
    m1, m3 = cfg.layers[1].mixer, cfg.layers[3].mixer
    assert state[1].shape == (m1.heads * m1.dim * m1.vdim + 3 * (2 * m1.kv_heads * m1.dim + m1.heads * m1.vdim),)
    assert state[3].shape == (m3.heads * m3.dim * m3.vdim,)
    assert state["after_embedding.0"].dtype == torch.int32 and state["after_embedding.0"].shape == ()
    man = CacheManager(kv, state, 16, 8, 4, allocate=False)
    assert len(man.groups) == 1 and man.groups[0].window == 21
    rc = man.open("a")
    man.extend(rc, 60)
    man.commit(rc, 60)
    assert rc.page_base[0] == (60 - 21 + 1) // 8          # pages before the wider window went back to the pool
    man.close(rc)
    man.assert_balanced()


def test_scaled_rotary_constants_match_plain():
    for dims, base, sc in ((16, 5e5, dict(factor=6.0, original=1024, fast=16.0, slow=2.0)), (8, 1e4, dict(factor=8.0, original=16, fast=4.0, slow=0.5)),
                           (32, 5e5, dict(factor=2.5, original=100, fast=20.0, slow=3.0))):
        rope = ScaledRope(BuildContext(torch.float32, torch.device("cpu"), 16), dims, base, rotary_dim=dims, **sc)
        f, mag = plain.rotary_frequencies({"dims": dims, "base": base, "scaling": sc})
        assert torch.allclose(rope._inv_freq_cpu.double(), torch.tensor(f, dtype=torch.float64), rtol=1e-6)
        assert abs(rope.magnitude - mag) < 1e-12 and abs(mag - (0.1 * math.log(sc["factor"]) + 1)) < 1e-12
        assert f[0] == 1.0 and f[-1] < base ** (-2.0 * (dims // 2 - 1) / dims) * 1.0000001      # fast pairs kept, slow pairs slowed


def test_plain_is_causal_and_windowed():
    from tests.kogonex_tiny import make_model_dir, read_weights
    import tempfile
    from pathlib import Path
    tiny = KOGOS["kogo_a"]
    with tempfile.TemporaryDirectory() as tmp:
        w = read_weights(make_model_dir(Path(tmp), tiny))
    cfg = tiny["cfg"].to_dict()
    ids = random_tokens(40, tiny["cfg"].vocab_size, 8)
    full = plain.forward(cfg, w, ids)
    assert (full[:17] - plain.forward(cfg, w, ids[:17])).abs().max() < 1e-9
    # a key outside every window and no recurrent layer: the first token no longer matters
    import copy
    only_attn = copy.deepcopy(cfg)
    only_attn["layers"] = [only_attn["layers"][0]]
    only_attn["embedding"] = {}
    w0 = {k: v for k, v in w.items() if k.startswith(("l0.", "embed", "final", "head"))}
    a = plain.forward(only_attn, w0, ids)
    b = plain.forward(only_attn, w0, [ids[0] + 1] + ids[1:])
    assert (a[9:] - b[9:]).abs().max() < 1e-12 and (a[8] - b[8]).abs().max() > 1e-6       # window 9: position 8 still sees key 0


def test_plain_router_groups_and_identity():
    r = {"top": 2, "experts": 4, "groups": {"count": 3, "keep": 1}}
    z = torch.tensor([0.0, 0.1, 3.0, -1.0, 2.9, 2.8], dtype=torch.float64)
    picked = plain.route(r, z, torch.zeros(6, dtype=torch.float64))
    assert [e for e, _ in picked] == [2, 3]                # the group of the largest score; its second member although small
    picked = plain.route(r, z, torch.tensor([0, 0, -5.0, 0, 0, 0], dtype=torch.float64))
    assert [e for e, _ in picked] == [4, 5]                # the correction moves the choice, not the weights
    s = torch.softmax(z, -1)
    assert abs(float(picked[0][1]) - float(s[4])) < 1e-15
