"""The committed tile table (katago_b200/csrc/kb_tile_table.h, read through the C ABI; no GPU needed): every tensor-core
convolution shape of the benchmark configurations has a row, and the planner returns that row."""
import numpy as np

from katago_b200 import capi
from katago_b200 import modelfile as mf


def _pad64(c):
    return (c + 63) // 64 * 64


def _block_shapes(blocks, C, out):
    """(k, inC, outC) of the convolutions the engine launches for a block stack on C channels (merged convolutions as
    they are launched: regular|gpool, up|gate, q|k|v)."""
    for b in blocks:
        kind = b["kind"]
        if kind == "ordinary_block":
            mid = b["conv1"]["outC"]
            out.add((b["conv1"]["kY"], C, mid)); out.add((b["conv2"]["kY"], mid, C))
        elif kind == "gpool_block":
            reg, gp = b["regularConv"]["outC"], b["gpoolConv"]["outC"]
            out.add((b["regularConv"]["kY"], C, reg + gp)); out.add((b["finalConv"]["kY"], reg, C))
        elif kind == "nested_bottleneck_block":
            mid = b["preConv"]["outC"]
            out.add((1, C, mid)); _block_shapes(b["blocks"], mid, out); out.add((1, mid, C))
        elif kind == "transformer_attention_block":
            qkv = b["heads"] * b["qDim"] + b["kvHeads"] * b["qDim"] + b["kvHeads"] * b["vDim"]
            out.add((1, C, qkv)); out.add((1, b["heads"] * b["vDim"], C))
        elif kind == "transformer_ffn_block":
            out.add((1, C, 2 * b["ffnC"])); out.add((1, b["ffnC"], C))
        else:
            raise AssertionError(kind)


def _net_shapes(tree):
    t = tree["trunk"]
    C = t["trunkC"]
    out = {(t["initialConv"]["kY"], _pad64(t["initialConv"]["inC"]), C)}
    _block_shapes(t["blocks"], C, out)
    p, v = tree["policyHead"], tree["valueHead"]
    out.add((1, C, p["p1Conv"]["outC"] + p["g1Conv"]["outC"] + v["v1Conv"]["outC"]))
    return out


def test_every_benchmark_shape_has_a_row_and_the_planner_returns_it():
    rows = {(r["k"], r["in_c"], r["out_c"]): r for r in capi.tile_table()}
    assert len(rows) == len(capi.tile_table()), "duplicate shape in the tile table"
    nets = dict(b18c384nbt=mf.make_b18c384nbt(), b28c512nbt=mf.make_b28c512nbt(), transformer=mf.make_transformer(),
                transformer_relbias=mf.make_transformer_relbias())
    for name, tree in nets.items():
        for (k, ic, oc) in sorted(_net_shapes(tree)):
            assert (k, ic, oc) in rows, f"{name}: convolution {k}x{k} {ic}->{oc} has no row in the tile table"
            plan = capi.tile_plan(k, ic, oc)
            row = rows[k, ic, oc]
            assert plan["from_table"]
            assert {x: plan[x] for x in ("bn", "pair", "epi_warps", "epi_warps_res", "chain")} == {x: row[x] for x in ("bn", "pair", "epi_warps", "epi_warps_res", "chain")}


def test_rows_are_consistent_and_other_shapes_fall_back():
    for r in capi.tile_table():
        assert r["k"] in (1, 3) and r["in_c"] % 64 == 0 and r["out_c"] % r["bn"] == 0 and r["bn"] % 16 == 0 and 16 <= r["bn"] <= 256
        assert r["epi_warps"] in (2, 3) and r["epi_warps_res"] in (2, 3) and r["pair"] in (0, 1)
        assert not (r["chain"] and (r["k"] != 3 or r["pair"])), r   # multi-layer launches: 3x3 convolutions on single CTAs
        assert not (r["pair"] and r["bn"] % 32), r
    p = capi.tile_plan(3, 320, 320)   # not a benchmark shape
    assert not p["from_table"] and p["bn"] == 160 and p["pair"] == 0 and p["chain"] == 1
    p = capi.tile_plan(1, 128, 96)
    assert not p["from_table"] and p["bn"] == 96 and p["epi_warps_res"] == 3
