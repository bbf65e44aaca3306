"""Vagulorn without a GPU: its configuration, the model as data, what its layers ask of the cache
manager (blocks of positions give pages back, kept first keys hold them), and properties of the plain
implementation itself."""

import copy

import pytest
import torch

from acorninfer_b200.cache.manager import CacheManager
from acorninfer_b200.config.model_config import ConfigError, VagulornConfig
from acorninfer_b200.models.decoder import Decoder, expected_tensors
from acorninfer_b200.parts.base import KVNeeds
from acorninfer_b200.registry import config_from_dict, spec_for
from tests.plain import vagulorn as plain
from tests.tiny import random_tokens
from tests.vagulorn_tiny import VAGU_LONG, VAGUS, make_model_dir, read_weights


@pytest.mark.parametrize("name", list(VAGUS))
def test_config_round_trip_and_registry(name):
    cfg = VAGUS[name]["cfg"]
    raw = cfg.to_dict()
    assert raw["architecture"] == "Vagulorn" and len(raw["layers"]) == len(cfg.layers)
    again = config_from_dict(raw)
    assert isinstance(again, VagulornConfig) and again == cfg


def test_config_errors_name_the_key():
    raw = VAGUS["vagu_a"]["cfg"].to_dict()
    for path, value, word in ((("layers", 0, "type"), "conv_mixer", "type"), (("layers", 0, "mixer", "rot", "dims"), 7, "rot.dims"),
                              (("layers", 1, "mixer", "groups"), 4, "groups"), (("layers", 2, "mixer", "right", "decay"), [0.5], "decay"),
                              (("layers", 2, "mixer", "left", "vdim"), 12, "vdim"), (("layers", 0, "mlp", "kind"), "moe", "kind"),
                              (("layers", 0, "mixer", "mask", "size"), 0, "mask.size"), (("norm", "eps"), 0.0, "eps")):
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
    cfg = VAGUS["vagu_a"]["cfg"]
    spec = spec_for(cfg)
    assert [ls.mixer.kind for ls in spec.layers] == ["attention", "state_space", "side_by_side", "state_space"]
    assert all(ls.block.kind == "parallel" and set(ls.norms) == {"input"} for ls in spec.layers)
    assert spec.layers[2].feed_forward is None and spec.head is None and spec.embedding_scale == 3.0
    names = expected_tensors(spec)
    for n in ("embed", "final.norm", "final.norm.b", "l0.norm1", "l0.norm1.b", "l0.mix.q.norm", "l0.mix.v", "l0.mlp.gate",
              "l1.mix.in", "l1.mix.conv.b", "l1.mix.A_log", "l1.mix.D", "l2.mix.left.g", "l2.mix.left.k.norm", "l2.mix.right.norm",
              "l2.mix.right.g", "l3.mix.dt_bias"):
        assert n in names, n
    assert "l2.mix.left.v" not in names and "l2.mlp.gate" not in names and "head" not in names
    assert names["l1.mix.in"].shape == (2 * 60 + 2 * 3 * 7 + 6, 72) and names["l1.mix.conv"].shape == (60 + 42, 4)
    assert names["l0.mix.o"].shape == (72, 4 * 20) and names["l2.mix.left.g"].shape == (3, 72)
    dec = Decoder(spec, torch.float32, "cpu", page_size=8)
    kv, state = dec.cache_needs()
    assert kv[0] == KVNeeds(2, 12, None, chunk=11, value_dim=20)
    assert kv[2] == KVNeeds(1, 10, 9, keep_first=3) and set(kv) == {0, 2}
    # state: S of all heads and the convolution's memory; beside attention, the linear attention's S alone
    assert state[1].shape == (6 * 7 * 10 + 3 * (60 + 42),) and state[3].shape == (2 * 20 * 24,)
    assert state[2].shape == (2 * 6 * 14,)
    # rotary settings: one encoding per distinct (head size, rotated entries, base, pairing)
    assert len(spec.positions) == 2


def test_pages_of_blocks_are_given_back_and_kept_first_keys_hold_theirs():
    needs = {0: KVNeeds(1, 8, None, chunk=20), 1: KVNeeds(1, 8, 12, keep_first=3), 2: KVNeeds(1, 8, 12)}
    m = CacheManager(needs, {}, 64, 4, 2, allocate=False)
    rc = m.open("a")
    for length in (7, 19, 20, 21, 45, 60, 61):
        m.extend(rc, length)
        m.commit(rc, length)
        g_blocks, g_kept, g_window = (m.group_of(e) for e in (0, 1, 2))
        # a later query at position >= length starts its block at length - length % 20
        assert rc.page_base[g_blocks] == (length - length % 20) // 4
        assert rc.page_base[g_kept] == 0 and len(rc.tables[g_kept]) == -(-length // 4)
        assert rc.page_base[g_window] == max(0, length - 12 + 1) // 4
    m.close(rc)
    m.assert_balanced()
    assert m.peak_pages(200, 16)[0] == -(-(20 + 16) // 4) + 1 and m.peak_pages(200, 16)[1] == 50


def test_plain_masks_and_recurrences():
    ok = plain.visible(12, "blocks", 5)
    assert ok[4, 0] and not ok[5, 4] and ok[9, 5] and not ok[10, 9] and ok[11, 10] and not ok[3, 4]
    ok = plain.visible(12, "window", 3, keep_first=2)
    assert ok[11, 9] and not ok[11, 8] and ok[11, 1] and ok[11, 0] and not ok[11, 2] and ok[2, 0] and not ok[5, 6]
    assert plain.visible(5, None, 0).sum() == 15
    # the selective recurrence with constant decays and unit steps is the decay recurrence
    g = torch.Generator().manual_seed(0)
    T, H, N, V = 9, 2, 3, 4
    k, q, v = (torch.randn(T, H, n, generator=g, dtype=torch.float64) for n in (N, N, V))
    decay = torch.tensor([0.5, 0.9], dtype=torch.float64)
    a = plain.decay_recurrence(decay, k, v, q)
    b = plain.selective_recurrence(decay[None].expand(T, H), torch.ones(T, H, dtype=torch.float64), k, q, v,
                                   torch.zeros(H, dtype=torch.float64))
    assert (a - b).abs().max() < 1e-12
    # ... and equals the sum over earlier tokens of decay^(t - s) (q_t . k_s) v_s
    t = 6
    direct = sum(decay[:, None] ** (t - s) * (q[t] * k[s]).sum(-1, keepdim=True) * v[s] for s in range(t + 1))
    assert (a[t] - direct).abs().max() < 1e-12
    # rotation keeps lengths and leaves the entries beyond the rotated part alone
    x = torch.randn(7, 2, 10, generator=g, dtype=torch.float64)
    for inter in (False, True):
        y = plain.rotate(x, 100.0, 6, inter)
        assert (y[..., 6:] == x[..., 6:]).all() and (y.norm(dim=-1) - x.norm(dim=-1)).abs().max() < 1e-12
        assert (y[0] - x[0]).abs().max() == 0
    # the convolution sees nothing before the first token, and its last tap is the current token's
    xs = torch.randn(5, 3, generator=g, dtype=torch.float64)
    taps = torch.tensor([[0.0, 0.0, 2.0]] * 3, dtype=torch.float64)
    assert (plain.causal_conv(xs, taps, torch.zeros(3, dtype=torch.float64)) - 2 * xs).abs().max() == 0


def test_plain_model_is_causal_and_sensitive_to_far_tokens(tmp_path):
    """Changing a token changes no earlier position; through the recurrent states it reaches positions far
    beyond every block and window."""
    tiny = VAGU_LONG
    d = make_model_dir(tmp_path, tiny)
    w = read_weights(d)
    toks = random_tokens(220, tiny["cfg"].vocab_size, 1)
    other = list(toks)
    other[30] = (other[30] + 1) % tiny["cfg"].vocab_size
    a = plain.forward(tiny["cfg"].to_dict(), w, toks)
    b = plain.forward(tiny["cfg"].to_dict(), w, other)
    assert (a[:30] - b[:30]).abs().max() == 0 and (a[30] - b[30]).abs().max() > 1e-3
    assert (a[215] - b[215]).abs().max() > 1e-9


def test_long_rows_are_cut_into_segments_only_where_the_device_is_not_full():
    from acorninfer_b200.kernels.ops import SCAN_MAX_SEGMENTS, SCAN_MIN_SEGMENT, scan_segments
    assert scan_segments(1, 64, 32, 128, 64) == (0, 1) and scan_segments(100, 1, 32, 128, 64) == (0, 1)
    seg, nseg = scan_segments(2048, 1, 32, 128, 64)
    assert 2 <= nseg <= SCAN_MAX_SEGMENTS and seg >= SCAN_MIN_SEGMENT and seg * nseg >= 2048
    assert scan_segments(2048, 64, 32, 128, 64) == (0, 1)            # 64 rows of 32 heads fill the device themselves
    seg, nseg = scan_segments(130, 1, 2, 16, 16)
    assert nseg == 2 and seg == 65
