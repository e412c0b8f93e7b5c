"""Parts and bookkeeping that need no GPU: refusals at build time, cache needs with tensors of any
per-token shape, the grouping of the forward pass into graph-safe runs, the logger."""
import io

import pytest
import torch

from conftest import TINY_B


def _runtime():
    from oracle_engine_b200.engine.runtime import Runtime
    return Runtime(torch.float32, torch.device("cpu"))


def test_attention_refuses_head_sizes_when_it_is_built():
    from oracle_engine_b200.parts.registry import MIXERS
    from oracle_engine_b200.parts import attention  # noqa: F401
    base = {"hidden_size": 64, "num_heads": 4, "num_kv_heads": 2, "position": None}
    MIXERS.get("gqa_attention")({**base, "head_dim": 256}, "", _runtime())
    for hd in (272, 15, 0):
        with pytest.raises(ValueError, match="head_dim"):
            MIXERS.get("gqa_attention")({**base, "head_dim": hd}, "", _runtime())
    with pytest.raises(ValueError, match="multiple"):
        MIXERS.get("gqa_attention")({**base, "head_dim": 16, "num_heads": 5}, "", _runtime())


def test_cache_groups_take_tensors_of_any_per_token_shape():
    """A mixer that keeps one latent vector per token, or keys and values of different widths,
    declares them; the cache stores each per page as [*outer, PAGE, inner]."""
    from oracle_engine_b200.cache.kv_cache import KVCache, page_shape
    from oracle_engine_b200.parts.spec import CacheNeed, attention_cache_need
    assert page_shape((2, 8, 128)) == (2, 8, 64, 128) and page_shape((24,)) == (64, 24)
    latent = CacheNeed("full", (("latent", (24,)),))
    uneven = CacheNeed("window", (("k", (2, 16)), ("v", (2, 40))), 100)
    needs = [attention_cache_need(2, 16), latent, None, uneven, latent]
    c = KVCache(needs, max_tokens=256, max_seq_len=256, dtype=torch.float32, device="cpu")
    assert [g.entries for g in c.groups] == [[0], [1, 4], [3]]
    kv, lat, un = (c.storage_of(e) for e in (0, 1, 3))
    assert kv["kv"].shape == (4, 2, 2, 64, 16)
    assert lat["latent"].shape == (4, 64, 24) and c.storage_of(4)["latent"].shape == (4, 64, 24)
    assert lat["latent"].data_ptr() != c.storage_of(4)["latent"].data_ptr()          # a cache of its own per entry
    assert un["k"].shape == (4, 2, 64, 16) and un["v"].shape == (4, 2, 64, 40)
    assert latent.elements_per_token() == 24 and uneven.elements_per_token() == 112
    assert c.groups[1].bytes_per_page(4) == 2 * 64 * 24 * 4
    s = c.alloc_slot()
    c.reserve(s, 130)
    c.commit(s, 130)
    c.check()
    c.free_slot(s)
    c.check()
    for bad in (CacheNeed("full", ()), CacheNeed("full", (("a", (4,)), ("a", (4,)))), CacheNeed("full", (("a", (0,)),)),
                CacheNeed("ring", (("a", (4,)),))):
        with pytest.raises(ValueError):
            KVCache([bad], 128, 128, allocate=False)


def test_forward_pass_is_grouped_into_graph_safe_runs():
    from oracle_engine_b200 import LlamaConfig
    from oracle_engine_b200.models.llama import build_spec
    from oracle_engine_b200.parts.model import DecoderModel
    model = DecoderModel(build_spec(LlamaConfig.from_dict(TINY_B)), _runtime())
    assert model.stages() == [(True, 0, 3 + 2)]               # embedding, three layers, head: one graph
    model.layers[1].mixer.graph_safe = False                  # as a mixer that must run eagerly would say
    assert model.stages() == [(True, 0, 2), (False, 2, 3), (True, 3, 5)]
    model.head.graph_safe = False
    assert model.stages() == [(True, 0, 2), (False, 2, 3), (True, 3, 4), (False, 4, 5)]
    model.embedding.graph_safe = False
    assert model.stages()[0] == (False, 0, 1)


def test_parts_report_what_they_compute():
    from oracle_engine_b200 import LlamaConfig
    from oracle_engine_b200.models.llama import build_spec
    from oracle_engine_b200.parts.model import DecoderModel
    cfg = LlamaConfig.from_dict(TINY_B)
    model = DecoderModel(build_spec(cfg), _runtime())
    D, FF, H, KVH, hd, L, V = 192, 512, 6, 2, 32, 3, 384
    per_token = 2.0 * (D * (2 * H + 2 * KVH) * hd + 3 * D * FF)
    # two sequences: 5 tokens on an empty cache, 1 token on 9 cached ones; the head on 2 rows
    seen = (1 + 2 + 3 + 4 + 5) + 10
    want = L * (6 * per_token + 4.0 * H * hd * seen) + 2 * 2.0 * V * D
    assert model.step_flops([0, 9], [5, 1], 2) == want


def test_logger_levels_and_format():
    from oracle_engine_b200.utils.log import Logger
    out = io.StringIO()
    lg = Logger(out)
    lg.set_level("warn")
    lg.info("build", "not shown")
    lg.warn("cache", "nearly full")
    lg.error("engine", "a wait ran out")
    lines = out.getvalue().splitlines()
    assert len(lines) == 2
    assert lines[0][2] == ":" and lines[0].endswith("[WARN] [cache] nearly full")
    assert lines[1].endswith("[ERR] [engine] a wait ran out")
    lg.set_level("off")
    lg.error("x", "y")
    assert len(out.getvalue().splitlines()) == 2
    with pytest.raises(ValueError):
        lg.set_level("loud")
