"""The device timeline's host side: grouping CTA records into launches and the report (no GPU needed)."""

from __future__ import annotations

import io

import numpy as np

from acvram_b200.kernels import timeline as T


def rec(kernel, block, grid, t0, t1, marks=()):
    r = np.zeros(1, dtype=T.RECORD)
    r["kernel"], r["block"], r["grid"], r["t0"], r["t1"] = kernel, block, grid, t0, t1
    for i, m in enumerate(marks):
        r["mark"][0][i] = m
    return r


def test_records_are_grouped_into_launches_by_kernel_grid_and_block():
    # a product of 2 CTAs, a norm of 1 CTA that began while the product ran, then the same product again
    parts = [rec(1, 0, 2, 1000, 5000, (1500, 4000)), rec(1, 1, 2, 1100, 5200, (1600, 4100)),
             rec(2, 0, 1, 3000, 6000),
             rec(1, 0, 2, 6100, 9000, (6500, 8000)), rec(1, 1, 2, 6150, 9100, (6600, 8100))]
    records = np.concatenate(parts)
    records = records[np.argsort(records["t0"], kind="stable")]
    Ls = T.launches(records)
    assert [(L["kernel"], L["grid"], len(L["blocks"])) for L in Ls] == [(1, 2, 2), (2, 1, 1), (1, 2, 2)]
    assert (Ls[0]["begin"], Ls[0]["end"]) == (1000, 5200) and (Ls[2]["begin"], Ls[2]["end"]) == (6100, 9100)
    assert Ls[0]["events"]["first_full"] == [1500, 1600] and Ls[2]["events"]["last_mma"] == [8000, 8100]
    assert Ls[1]["events"] == {}


def test_report_names_kernels_and_shows_overlap_as_negative_gap():
    records = np.concatenate([rec(1, 0, 1, 0, 4000, (500, 3000)), rec(2, 0, 1, 2000, 5000), rec(4, 0, 1, 6000, 9000, (7000,))])
    out = io.StringIO()
    T.report(records, file=out)
    text = out.getvalue()
    lines = text.splitlines()
    assert lines[1].split()[0] == "gemm" and lines[2].split()[0] == "norm" and lines[3].split()[0] == "attn_decode"
    assert float(lines[2].split()[3]) == -2.0         # the norm began 2 us before the product ended
    assert float(lines[3].split()[3]) == 1.0          # the attention began 1 us after everything before it had ended
    assert "first_full:0.5..0.5" in lines[1] and "loop_done:1.0..1.0" in lines[3]
    assert "step: 9.0 us" in text
