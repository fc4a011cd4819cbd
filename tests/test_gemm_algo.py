"""Offline GEMM variant search: candidate enumeration, selection with injected timings, map round trip and lookup."""
import json

import pytest
import torch

from oslo_b200.ops import gemm_algo as ga


def test_candidates_and_keys():
    assert [a.label() for a in ga.candidates(4096, 4096, 4096)] == ["1cta-auto", "1cta-128x64", "1cta-128x128", "1cta-128x256", "2cta-256x256"]
    assert [a.label() for a in ga.candidates(128, 96, 64)] == ["1cta-auto", "1cta-128x64"]
    assert ga.m_bucket(1) == 1 and ga.m_bucket(4096) == 4096 and ga.m_bucket(4097) == 8192
    assert ga.shape_key(3000, 512, 256, 0, 1, "fp16", 2) == "4096x512x256:nt:fp16:b2"
    assert ga.parse_shapes(["16x32x64", "1,2,3"]) == [(16, 32, 64), (1, 2, 3)]
    with pytest.raises(ValueError):
        ga.parse_shapes(["16x32"])
    assert ga.model_shapes(2048, 8192, 16384, vocab=50304, tp=2) == [(16384, 3072, 2048), (16384, 2048, 1024), (16384, 4096, 2048),
                                                                     (16384, 2048, 4096), (16384, 25152, 2048)]


def test_search_picks_the_fastest_agreeing_variant_and_map_round_trips(tmp_path):
    cost = {"1cta-auto": 1.0, "1cta-128x64": 1.4, "1cta-128x128": 0.9, "1cta-128x256": 0.8, "2cta-256x256": 0.7}
    calls = []

    def run(m, n, k, algo):
        if algo.two_cta and n == 512:
            raise RuntimeError("refused")  # a variant may decline a shape

        def fn():
            calls.append(algo.label())
            out = torch.ones(2, 2)
            if algo.block_n == 256 and n == 512:
                out = out * 3  # a variant with a wrong result must not win
            fn.label = algo.label()
            return out

        fn.label = algo.label()
        return fn

    log = []
    amap = ga.search([(4096, 4096, 4096), (4096, 512, 4096), (64, 64, 64)], run=run, timer=lambda fn: cost[fn.label], log=log.append)
    assert amap.get(4096, 4096, 4096) == ga.Algo(True, 0)
    assert amap.get(4096, 512, 4096) == ga.Algo(False, 128)  # 2cta refused, 128x256 wrong
    assert amap.get(64, 64, 64) == ga.Algo(False, 0)  # tie at 1.0 vs 1.4: the built-in choice
    assert any("refused" in line for line in log) and any("differs" in line for line in log)
    e = amap.entries[ga.shape_key(4096, 4096, 4096)]
    assert abs(e["tflops"] - 2 * 4096 ** 3 / 0.7e-3 / 1e12) < 1e-6 and len(e["timings_ms"]) == 5
    # bucketed lookup: 3000 rows fall into the 4096 bucket; a 2-CTA winner is not handed to a shape it cannot run
    assert amap.get(3000, 4096, 4096) == ga.Algo(True, 0)
    small = ga.AlgoMap()
    small.set(ga.shape_key(200, 512, 512), ga.Algo(True, 0), 1.0, 1.0)
    assert small.get(200, 512, 512) is None and small.get(256, 512, 512) == ga.Algo(True, 0)
    assert amap.get(4096, 4096, 4096, b_mn=1) is None and amap.get(4096, 4096, 2048) is None
    path = str(tmp_path / "algo.json")
    amap.save(path)
    again = ga.AlgoMap.load(path)
    assert again.entries == amap.entries
    raw = json.load(open(path))
    raw["version"] = 99
    json.dump(raw, open(path, "w"))
    with pytest.raises(ValueError):
        ga.AlgoMap.load(path)


def test_lookup_follows_the_loaded_map(tmp_path):
    amap = ga.AlgoMap()
    amap.set(ga.shape_key(1024, 1024, 1024), ga.Algo(False, 64), 0.1, 2.0 * 1024 ** 3)
    path = str(tmp_path / "m.json")
    amap.save(path)
    try:
        assert ga.load(path) is not None
        assert ga.lookup(1024, 1024, 1024, 0, 0, torch.bfloat16, 1) == ga.Algo(False, 64)
        assert ga.lookup(1024, 1024, 1024, 0, 0, torch.float16, 1) is None
    finally:
        ga.load(None)
    assert ga.lookup(1024, 1024, 1024, 0, 0, torch.bfloat16, 1) is None


@pytest.mark.gpu
def test_search_on_device_and_gemm_uses_the_map(tmp_path):
    from oslo_b200.ops.gemm import gemm

    amap = ga.search([(512, 512, 1024)], iters=3, log=lambda s: None)
    algo = amap.get(512, 512, 1024)
    assert algo is not None and len(amap.entries[ga.shape_key(512, 512, 1024)]["timings_ms"]) >= 4
    forced = ga.AlgoMap()
    forced.set(ga.shape_key(512, 512, 1024), ga.Algo(False, 64), 1.0, 1.0)
    path = str(tmp_path / "f.json")
    forced.save(path)
    a = torch.randn(512, 1024, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(512, 1024, device="cuda", dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    try:
        ga.load(path)
        out = gemm(a, b)
    finally:
        ga.load(None)
    assert (out.float() - ref).abs().max() < 0.02 * ref.abs().max()
