"""The tiling choice of the tensor-core path (tile shape, slabs per slot, cut of the contraction),
checked on the host through hc_plan_product: the launch code calls the same routine."""
import ctypes

import numpy as np
import pytest

from honeycrisp_b200 import _lib as L

F16, F32 = 0, 1
SMS = 148


def plan(dtype, count, rows, inner, cols, ta=False, tb=False, to=False, sms=SMS, diagnostics=False):
    info = L.PlanInfo()
    st = L.load(diagnostics).hc_plan_product(dtype, count, int(ta), int(tb), int(to), rows, inner, cols, sms, ctypes.byref(info))
    assert st == L.HC_OK, st
    return info


def test_benchmark_configurations():
    c2 = plan(F16, 1, 8192, 8192, 8192, tb=True)
    assert (c2.tile_m, c2.tile_n, c2.ctas_per_tile, c2.parts) == (256, 512, 2, 1)
    assert c2.tiles == 32 * 16 and c2.workspace_bytes == 0
    c3 = plan(F16, 64, 2048, 128, 2048, tb=True)
    assert (c3.tile_m, c3.tile_n, c3.parts, c3.tiles) == (256, 256, 1, 64 * 64)
    c5 = plan(F32, 1, 16384, 16384, 16384)
    assert (c5.tile_m, c5.tile_n, c5.parts) == (256, 256, 1)
    c1 = plan(F32, 1, 1024, 1024, 1024)
    assert (c1.tile_m, c1.tile_n, c1.parts) == (256, 64, 1)      # one wave either way: spread over more SMs


def test_small_products_take_small_pair_tiles():
    assert (plan(F16, 1, 512, 512, 512, tb=True).tile_n, plan(F16, 1, 1536, 1536, 1536, tb=True).tile_n) == (64, 128)
    assert plan(F16, 1, 2048, 2048, 2048, tb=True).tile_n == 256
    # 32 columns of B per CTA cannot be cut out of an MN-major (not transposed) float16 operand
    assert plan(F16, 1, 512, 512, 512, tb=False).tile_n == 128
    # at most 128 rows: no CTA pairs
    assert plan(F16, 1, 128, 4096, 4096, tb=True).ctas_per_tile == 1
    # two k slabs per pipeline slot on the small float16 shapes only
    assert plan(F16, 1, 512, 512, 512, tb=True).slabs_per_slot == 2
    assert plan(F16, 1, 4096, 4096, 4096, tb=True).slabs_per_slot == 1
    assert plan(F32, 1, 512, 512, 512).slabs_per_slot == 1


def test_long_contractions_over_few_outputs_are_cut():
    p = plan(F16, 1, 512, 4096, 512, tb=True)
    assert p.parts >= 2 and p.workspace_bytes == p.parts * 512 * 512 * 4
    assert p.tiles <= SMS // 2 * 2                     # the cut fills at most one wave
    assert plan(F32, 1, 512, 4096, 512).parts >= 2
    assert plan(F16, 1, 8192, 8192, 8192, tb=True).parts == 1    # a full wave needs no cut
    assert plan(F16, 1, 512, 256, 512, tb=True).parts == 1       # too short to cut


def test_switches(monkeypatch):
    """The HC_TC_* switches exist in the diagnostics build only; the shipped library ignores them."""
    dplan = lambda *a, **k: plan(*a, diagnostics=True, **k)
    monkeypatch.setenv("HC_TC_SPLITS", "1")
    assert dplan(F16, 1, 512, 4096, 512, tb=True).parts == 1
    assert plan(F16, 1, 512, 4096, 512, tb=True).parts >= 2
    monkeypatch.setenv("HC_TC_SPLITS", "5")
    assert dplan(F16, 1, 512, 4096, 512, tb=True).parts == 5
    monkeypatch.delenv("HC_TC_SPLITS")
    for forced, tile in {1: (256, 512), 2: (256, 256), 3: (128, 256), 4: (128, 128), 5: (256, 128), 6: (256, 64)}.items():
        monkeypatch.setenv("HC_TC_SHAPE", str(forced))
        p = dplan(F16, 1, 1024, 4096, 2048, tb=True)
        assert (p.tile_m, p.tile_n) == tile, forced
    monkeypatch.setenv("HC_TC_SHAPE", "1")
    assert dplan(F16, 1, 1024, 512, 512, tb=True).tile_n != 512    # a shape the product does not admit is ignored
    monkeypatch.setenv("HC_TC_SHAPE", "6")
    assert plan(F16, 1, 8192, 8192, 8192, tb=True).tile_n == 512    # shipped library: no switches


def test_every_part_has_work_and_the_parts_cover_the_contraction():
    rng = np.random.default_rng(0)
    for _ in range(400):
        dtype = int(rng.integers(0, 2))
        rows, cols = (int(rng.integers(1, 40)) * 8 for _ in range(2))
        inner = int(rng.integers(1, 2200)) * 8
        count = int(rng.integers(1, 4))
        flags = [bool(x) for x in rng.integers(0, 2, 3)]
        p = plan(dtype, count, rows, inner, cols, *flags)
        slab = 64 if dtype == F16 else 32
        kslots = -(-(-(-inner // slab)) // p.slabs_per_slot)
        assert p.parts >= 1 and p.slots_per_part >= 1
        assert p.parts * p.slots_per_part >= kslots, (rows, inner, cols, p.parts, p.slots_per_part)
        assert (p.parts - 1) * p.slots_per_part < kslots, (rows, inner, cols, p.parts, p.slots_per_part)
        assert p.workspace_bytes <= 256 << 20
        assert (p.workspace_bytes > 0) == (p.parts > 1)
        out_rows, out_cols = (cols, rows) if flags[2] else (rows, cols)
        assert p.tiles == -(-out_rows // p.tile_m) * -(-out_cols // p.tile_n) * count * p.parts


def test_more_sms_never_mean_fewer_tiles_per_wave():
    # the same product on a smaller device: still a valid plan
    for sms in (2, 16, 74, 132, 148, 160):
        p = plan(F16, 1, 4096, 4096, 4096, tb=True, sms=sms)
        assert p.tile_m in (128, 256) and p.tile_n in (64, 128, 256, 512)


def test_invalid_arguments():
    info = L.PlanInfo()
    lib = L.load()
    assert lib.hc_plan_product(F16, 1, 0, 0, 0, 0, 8, 8, SMS, ctypes.byref(info)) == L.HC_ERR_INVALID_ARGUMENT
    assert lib.hc_plan_product(7, 1, 0, 0, 0, 8, 8, 8, SMS, ctypes.byref(info)) == L.HC_ERR_INVALID_ARGUMENT
    assert lib.hc_plan_product(F16, 1, 0, 0, 0, 8, 8, 8, SMS, None) == L.HC_ERR_INVALID_ARGUMENT
