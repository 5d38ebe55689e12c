"""Launch planning is pure host arithmetic (ffn_int4_describe_plan): checked here, without a GPU, for
the benchmark shapes, their tensor-parallel slices and a few shapes no GPU test runs, against the
limits the kernels rely on (shared memory, pipeline depth, thread layout, coverage of rows)."""
import ctypes

import pytest

from haskell_infer_demo_b200 import lib as L

SMS, SMEM = 148, 232448            # B200: SM count, opt-in shared memory per block
SHAPES = [(1024, 3072), (2560, 9728), (5120, 17408), (8192, 28672), (4096, 14336), (5120, 34816)]


def plan(tokens, hidden, inter, sms=SMS, smem=SMEM):
    buf = ctypes.create_string_buffer(1024)
    st = L.load().ffn_int4_describe_plan(tokens, hidden, inter, sms, smem, buf, len(buf))
    assert st == 0, L.load().ffn_int4_last_error()
    text = buf.value.decode()
    fields = dict(kv.split("=", 1) for kv in text.split() if "=" in kv)
    return {k: (int(v) if v.lstrip("-").isdigit() else v) for k, v in fields.items()}


@pytest.mark.parametrize("hidden,inter", SHAPES)
@pytest.mark.parametrize("tp", [1, 2, 4, 8])
@pytest.mark.parametrize("tokens", [1, 2])
def test_fused_plan_respects_the_kernel_limits(hidden, inter, tp, tokens):
    local = inter // tp
    if local % 128:
        pytest.skip("the split is not a whole number of groups; the loader refuses it")
    p = plan(tokens, hidden, local)
    if p["kernel"] != "fused":
        assert p["kernel"] in ("tcgen05_pair", "mma_pair", "generic")       # a shape the single-launch kernel does not take
        return
    assert p["grid"] == SMS and p["threads"] == 608
    assert p["smem"] <= SMEM and p["stages"] >= 2
    assert p["act_bytes"] >= tokens * local * 2
    for ph, k in (("p1", hidden), ("p2", local)):
        ct, rg, cit = p[f"{ph}_ct"], p[f"{ph}_rg"], p[f"{ph}_cit"]
        assert ct % 16 == 0 and ct * rg <= 544 and ct * cit >= k // 32      # whole half-warps; every 16-byte chunk has a thread
        assert tokens * cit <= 2                                           # prepared activation slices a thread can hold
    assert p["p1_pairs_per_tile"] == p["p1_rg"] * p["p1_jt"] and p["p1_jt"] <= 2
    assert p["p2_rows_per_tile"] == p["p2_rg"] * p["p2_jt"] and p["p2_jt"] <= 4
    # a tile (both halves of a pair tile, or the down rows) fits the stage it is copied into
    assert 2 * p["p1_pairs_per_tile"] * (hidden // 2) <= p["stage_bytes"]
    assert p["p2_rows_per_tile"] * (local // 2) <= p["stage_bytes"]


def test_headline_shape_uses_all_of_shared_memory():
    p = plan(1, 5120, 17408)
    assert (p["stages"], p["stage_bytes"], p["p1_pairs_per_tile"], p["p2_rows_per_tile"]) == (3, 64768, 12, 6)
    assert SMEM - p["smem"] < p["stage_bytes"]               # no room for another stage was left unused


@pytest.mark.parametrize("tokens", [3, 8, 16, 17, 32, 33, 64])
@pytest.mark.parametrize("hidden,inter,tp", [(5120, 17408, 1), (5120, 17408, 8), (1024, 3072, 1), (2560, 9728, 2)])
def test_batched_plan(tokens, hidden, inter, tp):
    local = inter // tp
    assert plan(tokens, hidden, local)["kernel"] == ("tcgen05_pair" if tokens > 16 and 2 * (local // 64) >= SMS else "mma_pair")   # the default choice
    old = L.load().ffn_int4_set_batched_kernel(1)
    try:
        p = plan(tokens, hidden, local)
    finally:
        L.load().ffn_int4_set_batched_kernel(old)
    assert p["kernel"] == "mma_pair"
    assert p["token_tiles"] * 8 >= tokens and p["token_tiles"] in (1, 2, 4, 8)
    assert p["smem"] * p["ctas_per_sm"] <= SMEM and p["stages"] >= 2
    assert p["gate_up_ctas"] * 64 == local and p["down_ctas"] == (hidden // 128) * p["down_k_splits"]
    assert 1 <= p["down_k_splits"] <= 8 and p["down_k_splits"] * 2 <= max(local // 128, 2)
    # the split count never leaves the last wave of CTAs emptier than no split would
    slots = SMS * p["ctas_per_sm"]
    eff = lambda u: u / (-(-u // slots) * slots)
    assert eff(p["down_ctas"]) >= eff(hidden // 128) - 1e-9
    # the tcgen05 pair, forced
    old = L.load().ffn_int4_set_batched_kernel(0)
    try:
        p = plan(tokens, hidden, local)
    finally:
        L.load().ffn_int4_set_batched_kernel(old)
    assert p["kernel"] == "tcgen05_pair"
    assert p["token_columns"] >= tokens and p["token_columns"] % 16 == 0 and p["token_columns"] <= 64
    assert p["smem"] <= SMEM and p["stages"] >= 2 and p["threads"] == 544 and p["operand_buffers"] == 4
    assert p["accumulator_buffers"] * p["token_columns"] + p["operand_buffers"] * 64 <= p["tmem_columns"] == 512
    assert p["gate_up_units"] * 64 == local and p["gate_up_ctas"] == min(p["gate_up_units"], SMS)
    assert p["down_units"] == (hidden // 128) * p["down_k_splits"] <= SMS
    assert 1 <= p["down_k_splits"] <= 8 and p["down_k_splits"] * 2 <= max(local // 128, 2)


def test_long_batches_run_in_blocks_of_64_and_small_devices_fall_back():
    assert plan(100, 5120, 17408)["passes"] == 2
    assert plan(4, 5120, 17408, smem=40 * 1024)["kernel"] == "generic"   # no room for the pair's pipeline
    lib = L.load()
    buf = ctypes.create_string_buffer(256)
    assert lib.ffn_int4_describe_plan(1, 5120, 100, SMS, SMEM, buf, 256) == -4      # not whole groups
    assert lib.ffn_int4_describe_plan(0, 5120, 17408, SMS, SMEM, buf, 256) == -4
    assert lib.ffn_int4_describe_plan(1, 5120, 17408, SMS, SMEM, buf, 8) == -4      # buffer too small


def test_smaller_shared_memory_means_fewer_stages_or_another_kernel():
    big = plan(1, 5120, 17408)
    small = plan(1, 5120, 17408, smem=170000)
    assert small["kernel"] == "fused" and small["stages"] < big["stages"]
    assert plan(1, 5120, 17408, smem=100 * 1024)["kernel"] != "fused"


@pytest.mark.parametrize("padded", [16, 32, 48, 64])
def test_tile_order_is_a_bijection_with_the_documented_structure(padded):
    """The activation layout of the tcgen05 pair (host arithmetic): every (token, k) of a [padded, K] bf16
    matrix gets its own 2-byte slot in [0, padded * K * 2); a 64-wide K block of all tokens is one
    contiguous padded * 128-byte slice (what one bulk copy per stage brings in); a token's 8 consecutive
    values of K share one 16-byte piece in the order (0,4),(1,5),(2,6),(3,7); pieces are swizzled by
    token & 7 inside the token's 128-byte row."""
    lib = L.load()
    K = 256
    off = [[lib.ffn_int4_tile_order_offset(n, k, padded) for k in range(K)] for n in range(padded)]
    flat = sorted(o for row in off for o in row)
    assert flat == list(range(0, padded * K * 2, 2))
    for n in (0, 5, padded - 1):
        for k0 in range(0, K, 64):
            block = [off[n][k] for k in range(k0, k0 + 64)]
            assert min(block) // (padded * 128) == k0 // 64 == max(block) // (padded * 128)          # the K block's slice
            row = (k0 // 64) * padded * 128 + (n // 8) * 1024 + (n % 8) * 128
            assert all(row <= o < row + 128 for o in block)                                          # the token's row in it
            for c in range(8):
                piece = [off[n][k0 + 8 * c + e] for e in range(8)]
                base = row + ((c ^ (n % 8)) << 4)
                assert [p - base for p in piece] == [0, 4, 8, 12, 2, 6, 10, 14]                      # (0,4),(1,5),(2,6),(3,7)
    assert lib.ffn_int4_tile_order_offset(padded, 0, padded) == -1 and lib.ffn_int4_tile_order_offset(0, 0, 24) == -1


def test_timeline_tool_imports_and_refuses_without_a_gpu(monkeypatch):
    import sys

    import torch

    import haskell_infer_demo_b200.trace as trace
    if torch.cuda.is_available():
        pytest.skip("a GPU is present: the tool would run")
    monkeypatch.setattr(sys, "argv", ["trace", "decode"])
    with pytest.raises(SystemExit):
        trace.main()
