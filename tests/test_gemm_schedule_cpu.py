"""The tile kernel's schedule, checked without a GPU: fl_sm100_gemm_plan() gives the numbers a
launch would use, and the walk every role of a CTA makes over them (mirrored here from
gemm_sm100.cu's WorkWalk) must cover every K stage of every tile exactly once; a tile cut by the
stream-K part must have exactly two holders, neighbouring units, the head held by the earlier unit
(the first thing it does in that part) and the tail by the later one (the last thing it does), which
is what the kernel's workspace slots and its two-arrival counters rely on."""
import ctypes

import pytest

from libwaifu_b200 import flint as F

KINDS = {"half": 0, "bf16": 1, "e4m3": 2, "nvfp4": 3}


def plan(kind, m, n, k, sms, allow=1):
    out = (ctypes.c_int32 * 8)()
    F.check(F.lib().fl_sm100_gemm_plan(KINDS[kind], m, n, k, sms, allow, out))
    return dict(zip(("ctas", "block_n", "tiles", "num_kb", "units", "dp_rounds", "sk_tiles", "sk_first_tile"), out))


def walk(p, unit):
    """The items of one unit: (tile, kb0, kb1, partial, head). In the stream-K part: the head of the
    tile the unit's run ends in, the whole tiles inside the run, the tail of the tile it starts in."""
    items = []
    for r in range(p["dp_rounds"]):
        tile = r * p["units"] + unit
        if tile >= p["tiles"]:
            break
        items.append((tile, 0, p["num_kb"], False, False))
    if p["sk_tiles"] == 0:
        return items
    kb = p["num_kb"]
    total = p["sk_tiles"] * kb
    begin, end = total * unit // p["units"], total * (unit + 1) // p["units"]
    t, length = divmod(end, kb)
    if length:
        items.append((p["sk_first_tile"] + t, 0, length, True, True))
    whole = -(-begin // kb)
    while (whole + 1) * kb <= end:
        items.append((p["sk_first_tile"] + whole, 0, kb, False, False))
        whole += 1
    t, kb0 = divmod(begin, kb)
    if kb0:
        items.append((p["sk_first_tile"] + t, kb0, kb, True, False))
    return items


SHAPES = [("e4m3", 4352, 12288, 3072), ("e4m3", 4352, 3072, 12288), ("e4m3", 4096, 3072, 3072), ("e4m3", 8704, 9216, 3072),
          ("e4m3", 8704, 3072, 3072), ("e4m3", 8704, 12288, 3072), ("e4m3", 8704, 3072, 12288), ("nvfp4", 4352, 9216, 3072),
          ("bf16", 4096, 12288, 3072), ("e4m3", 1024, 12288, 3072), ("e4m3", 520, 328, 1024), ("e4m3", 130, 264, 208),
          ("e4m3", 8192, 3072, 64), ("e4m3", 300, 200, 256), ("half", 513, 64, 64), ("e4m3", 19200, 256, 512),
          ("e4m3", 2, 18432, 3072), ("e4m3", 77 * 256, 256, 8192), ("e4m3", 149 * 128, 128, 8192),
          ("e4m3", 2304, 2304, 6144), ("e4m3", 20480, 128, 6144), ("e4m3", 2250, 2312, 6160), ("nvfp4", 2304, 1728, 12288),
          ("bf16", 2304, 2304, 3072), ("e4m3", 5000, 5000, 16384),
          ("e4m3", 4352, 384, 12288), ("e4m3", 1024, 384, 12288), ("bf16", 512, 256, 8192), ("e4m3", 300, 200, 10368)]


@pytest.mark.parametrize("sms", [148, 132, 16, 2])
@pytest.mark.parametrize("kind,m,n,k", SHAPES)
def test_every_stage_of_every_tile_is_computed_once(kind, m, n, k, sms):
    p = plan(kind, m, n, k, sms)
    halves = p["sk_tiles"] > 0 and p["units"] == 2 * p["tiles"]  # few tiles, long K: every tile in two halves
    if halves:
        assert p["units"] <= sms // p["ctas"] and (p["dp_rounds"], p["sk_tiles"], p["sk_first_tile"]) == (0, p["tiles"], 0)
    else:
        assert p["units"] == min(p["tiles"], sms // p["ctas"])
        assert p["sk_tiles"] == 0 or p["sk_tiles"] >= p["units"]
    assert p["dp_rounds"] * p["units"] == p["sk_first_tile"] or p["sk_tiles"] == 0
    covered = {}
    holders = {}
    for u in range(p["units"]):
        items = walk(p, u)
        for index, (tile, kb0, kb1, partial, head) in enumerate(items):
            assert 0 <= tile < p["tiles"] and 0 <= kb0 < kb1 <= p["num_kb"]
            for kb in range(kb0, kb1):
                assert (tile, kb) not in covered, f"stage {kb} of tile {tile} computed twice"
                covered[(tile, kb)] = u
            if partial:
                # a part is the head (from stage 0) or the tail (to the last stage), never the middle
                assert (kb0 == 0) != (kb1 == p["num_kb"])
                assert head == (kb0 == 0)
                # the head is its unit's first item of the stream-K part, the tail its unit's last item
                if head:
                    assert index == p["dp_rounds"]
                else:
                    assert index == len(items) - 1
                holders.setdefault(tile, []).append((u, head))
    assert len(covered) == p["tiles"] * p["num_kb"]
    for tile, parts in holders.items():
        assert len(parts) == 2, f"tile {tile} is cut into {len(parts)} parts"
        (u0, h0), (u1, h1) = sorted(parts)
        assert h0 and not h1 and u1 == u0 + 1, f"tile {tile}: head in unit {u0} ({h0}), tail in unit {u1} ({h1})"
    # workspace bounds the kernel indexes: two slots per unit, a counter set per stream-K tile
    assert p["sk_tiles"] <= 2 * p["units"]


def test_stream_k_is_taken_where_it_saves_forty_stages_or_more():
    # the denoise step's down projection: 408 pair tiles on 74 pairs, 96 stages each; the last round
    # would be 38 / 74 full
    down = plan("e4m3", 8704, 3072, 12288, 148)
    assert (down["ctas"], down["block_n"], down["tiles"], down["units"], down["num_kb"]) == (2, 256, 408, 74, 96)
    assert (down["dp_rounds"], down["sk_tiles"], down["sk_first_tile"]) == (4, 112, 296)
    # 3072-deep tiles have 24 stages: never worth it
    up = plan("e4m3", 4352, 12288, 3072, 148)
    assert (up["tiles"], up["dp_rounds"], up["sk_tiles"]) == (816, 12, 0)
    # a long-K product whose last round is three quarters full: 23 stages to save, not taken
    assert plan("e4m3", 4352, 3072, 12288, 148)["sk_tiles"] == 0
    # without a workspace tiles stay whole
    assert plan("e4m3", 8704, 3072, 12288, 148, allow=0)["sk_tiles"] == 0
    assert plan("e4m3", 520, 328, 8192, 148)["sk_tiles"] == 0          # fewer tiles than units
    assert plan("e4m3", 2304, 2304, 6144, 148)["sk_tiles"] == 81        # what the GPU tests run
    # few tiles and a long K: every tile in two halves on twice as many units
    few = plan("e4m3", 4352, 384, 12288, 148)
    assert (few["tiles"], few["units"], few["dp_rounds"], few["sk_tiles"]) == (34, 68, 0, 34)
    assert plan("e4m3", 4352, 768, 12288, 148)["sk_tiles"] == 0          # 51 tiles: twice that does not fit 74 pairs
