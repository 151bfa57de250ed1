"""Launch plans of the configuration shapes, checked on the host (ztq_describe_plan is plain arithmetic: no GPU).

What the planner decides is what the benchmark numbers depend on: which kernel a shape gets, how many rows a stage
holds, how deep the ring is, how many tiles and passes the busiest CTA walks, how the tensor-core kernel cuts K.  These
tests pin the invariants every plan must keep and the choices the measurements were made with, for a B200 (148 SMs) and
for other SM counts (the plan must stay valid, not identical).
"""
import pytest

from ztensor_b200 import kernels as K

SMS = 148
SHAPES_8B = [(6144, 4096), (4096, 4096), (14336, 4096), (4096, 14336)]
SHAPES_70B = [(10240, 8192), (8192, 8192), (57344, 8192), (8192, 28672)]
SHARDS = [(10240 // w, 8192) for w in (2, 4, 8)] + [(8192, 8192 // w) for w in (2, 4, 8)] + \
         [(57344 // w, 8192) for w in (2, 4, 8)] + [(8192, 28672 // w) for w in (2, 4, 8)]


@pytest.mark.parametrize("fmt", ["q4_0", "iq4nl", "w4g", "q8_0"])
@pytest.mark.parametrize("n,k", SHAPES_8B + SHAPES_70B + SHARDS + [(11008, 4096), (300, 4096), (257, 1024)])
@pytest.mark.parametrize("sms", [148, 132, 64])
def test_gemv_plans_are_valid(fmt, n, k, sms):
    pl = K.describe_plan(fmt, n, k, 1, 128, sms)
    assert pl["kernel"] in ("stream", "pair")
    assert pl["stages"] >= 2 and pl["rows_per_stage"] >= 1
    assert pl["rt"] in (2, 4) and pl["rows_per_stage"] == pl["teams"] * pl["rt"]
    assert pl["rows_per_pass"] % pl["rows_per_stage"] == 0 and pl["rows_per_pass"] >= pl["rows_per_stage"]
    assert 1 <= pl["grid"] <= 2 * sms
    # every row has a home: the busiest CTA's tiles cover its share
    per_cta = -(-n // pl["grid"])
    assert pl["tiles_per_cta"] * pl["rows_per_stage"] >= per_cta
    assert pl["passes_per_cta"] * pl["rows_per_pass"] >= min(per_cta, pl["tiles_per_cta"] * pl["rows_per_stage"])
    if pl["kernel"] == "pair":
        assert fmt in ("q4_0", "w4g") and k >= 2048 and k % 64 == 0 and n >= 12 * sms
        assert pl["grid"] <= sms and pl["warps_per_team"] * pl["teams"] <= 16
        assert pl["warps_per_team"] * 32 * 64 >= k                     # a team spans K: 64 weights per lane
    else:
        assert pl["warps_per_team"] * pl["teams"] <= 16


def test_choices_the_measurements_were_made_with():
    # the headline kernel: merged gate|up of the 70B stack
    pl = K.describe_plan("w4g", 57344, 8192, 1, 128, SMS)
    assert pl["kernel"] == "pair" and pl["rt"] == 4 and pl["grid"] == SMS and pl["tiles_per_cta"] > pl["stages"]
    # long rows: the planes' shared memory becomes stages once every warp holds its activations
    assert K.describe_plan("w4g", 8192, 28672, 1, 128, SMS)["overlay_stages"] >= 1
    # fewer than a dozen rows per SM: the one-chunk kernel (8-rank QKV shard), also for rows shorter than 2048 weights
    assert K.describe_plan("w4g", 1280, 8192, 1, 128, SMS)["kernel"] == "stream"
    assert K.describe_plan("w4g", 8192, 1024, 1, 128, SMS)["kernel"] == "stream"
    # formats without a chunk-pair kernel
    for fmt in ("q8_0", "iq4nl", "ternary"):
        assert K.describe_plan(fmt, 11008 if fmt == "ternary" else 14336, 4096, 1, 128, SMS)["kernel"] == "stream"
    # scale rows that do not start on 16 bytes (86 groups of 4 bytes): the plain kernel, any alignment
    assert K.describe_plan("w4g", 4096, 11008, 1, 128, SMS)["kernel"] == "plain"
    # K-quants run in the chunk-pair kernel
    for fmt in ("q4_k", "q5_k", "q6_k"):
        assert K.describe_plan(fmt, 14336, 4096, 1, 128, SMS)["kernel"] == "pair"


@pytest.mark.parametrize("n,k", SHAPES_8B + SHAPES_70B + [(28672, 4096), (12800, 28672), (1000, 2048), (128, 512)])
@pytest.mark.parametrize("batch", [3, 8, 16, 32, 40])
@pytest.mark.parametrize("sms", [148, 132])
def test_tensor_core_plans_are_valid(n, k, batch, sms):
    pl = K.describe_plan("w4g_tc", n, k, batch, 128, sms)
    tiles, groups = -(-n // 128), k // 128
    assert pl["kernel"] == "tensor" and pl["row_tiles"] == tiles
    assert pl["columns"] in (8, 16, 32) and pl["columns"] >= min(batch, 32) or pl["columns"] == 32
    s = pl["k_slices"]
    assert 1 <= s <= 8 and groups % (4 * s) == 0 if s > 1 else s == 1      # slices of whole groups of four
    assert pl["groups_per_slice"] * s == groups
    assert pl["items"] == tiles * s and pl["grid"] == min(pl["items"], sms)
    assert pl["items_per_cta"] == -(-pl["items"] // pl["grid"])


def test_tensor_core_k_split_fills_the_sms_when_row_tiles_are_few():
    # 32 row tiles on 148 SMs: split; 448 row tiles: whole tiles
    assert K.describe_plan("w4g_tc", 4096, 4096, 16, 128, SMS)["k_slices"] >= 2
    assert K.describe_plan("w4g_tc", 57344, 8192, 8, 128, SMS)["k_slices"] == 1
    # K % 512 is what the kernel needs
    with pytest.raises(ValueError):
        K.describe_plan("w4g_tc", 4096, 4096 + 128, 16, 128, SMS)


def test_arguments_no_entry_point_accepts():
    for args in (("w4g", 0, 4096), ("w4g", 4096, 0), ("q4_0", 4096, 4096 + 16)):
        with pytest.raises(ValueError):
            K.describe_plan(args[0], args[1], args[2], 1, 128, SMS)
    with pytest.raises(ValueError):
        K.describe_plan("w4g", 4096, 4096, 0, 128, SMS)
