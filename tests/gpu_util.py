"""Helpers shared by the GPU parity tests: move oracle cases to the device,
call the library through its C ABI wrappers, compare with the tolerances the
library promises (BF16 output: max-abs 2e-2 and mean-abs 2e-3; LSE: 1e-3
relative)."""
import numpy as np
import torch

from oracle import dsv4_oracle as orc

OUT_MAX_ABS = 2e-2
OUT_MEAN_ABS = 2e-3
LSE_REL = 1e-3


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def bits_to_f32(bits):
    return orc.bf16_bits_to_f32(bits)


def out_to_f32(t):
    return t.float().cpu().numpy()


OUT_MAX_REL_PEAK = 5e-2      # largest error against the largest output of the tensor
OUT_MEAN_REL = 1e-2          # mean error against the mean output magnitude (BF16 rounding alone gives about 2e-3)


def check_out(got_f32, want_bits, what=""):
    want = bits_to_f32(want_bits)
    err = np.abs(got_f32 - want)
    assert np.isfinite(got_f32).all(), f"{what}: non-finite output"
    assert err.max() <= OUT_MAX_ABS, f"{what}: max-abs {err.max():.4g} > {OUT_MAX_ABS}"
    assert err.mean() <= OUT_MEAN_ABS, f"{what}: mean-abs {err.mean():.4g} > {OUT_MEAN_ABS}"
    # the absolute bounds say little where the outputs are small (long rows average many values): also bound the
    # errors against the size of the outputs themselves
    peak, mean = float(np.abs(want).max()), float(np.abs(want).mean())
    if peak > 0:
        assert err.max() <= OUT_MAX_REL_PEAK * peak + 1e-6, f"{what}: max-abs {err.max():.4g} > {OUT_MAX_REL_PEAK} x largest output {peak:.4g}"
        assert err.mean() <= OUT_MEAN_REL * mean + 1e-7, f"{what}: mean-abs {err.mean():.4g} > {OUT_MEAN_REL} x mean output {mean:.4g}"
    return float(err.max()), float(err.mean())


def check_lse(got, want, what=""):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    inf = np.isneginf(want)
    assert np.array_equal(np.isneginf(got), inf), f"{what}: -inf pattern differs"
    fin = ~inf
    if fin.any():
        rel = np.abs(got[fin] - want[fin]) / np.maximum(np.abs(want[fin]), 1.0)
        assert rel.max() <= LSE_REL, f"{what}: lse rel err {rel.max():.4g} > {LSE_REL}"


def csa_to_dev(case):
    return dict(q=dev(case.q, torch.bfloat16), kv_pool=dev(case.pool), block_table=dev(case.block_table),
                indices=dev(case.indices), kv_len=dev(case.kv_len), sm_scale=case.sm_scale)


def hca_to_dev(case):
    return dict(q=dev(case.q, torch.bfloat16), kv_pool=dev(case.pool), block_table=dev(case.block_table),
                kv_len=dev(case.kv_len), win_pool=dev(case.win), win_len=dev(case.win_len),
                sm_scale=case.sm_scale, attn_sink=None if case.sink is None else dev(case.sink))
