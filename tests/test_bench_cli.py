"""The bench CLI that mirrors the reference's ``bwmoe-bench`` and ``scripts/bench_matrix.py``: the CSV it
writes has that script's columns (scripts/bench_matrix.py:39-51) and its shape list (:15-25)."""

import csv

import pytest

from blackwell_moe_b200 import bench_cli


def test_shape_list_and_csv_columns_are_the_reference_matrix(tmp_path):
    assert list(bench_cli.SHAPES) == ["toy_E16", "olmoe_1B_7B", "qwen3_30B_A3B", "qwen3_moe_57B_14B", "mixtral_8x7B",
                                      "mixtral_8x22B_prefill", "mixtral_8x22B_decode", "deepseek_v2_lite",
                                      "deepseek_E128"]
    assert bench_cli.SHAPES["mixtral_8x7B"] == dict(T=4096, D=4096, E=8, K=2, H=14336)

    def fake_runner(T, D, E, K, H, **kw):
        return [bench_cli.BenchResult("fp8_sm100", 2.0, T / 2e-3, 10.0), bench_cli.BenchResult("fp8_sm100_graph", 1.0, T / 1e-3, 10.0)]

    rows = bench_cli.matrix_rows(["toy_E16", "deepseek_v2_lite"], runner=fake_runner)
    path = bench_cli.write_csv(rows, tmp_path / "bench_results" / "matrix.csv")
    with open(path) as f:
        got = list(csv.DictReader(f))
    assert list(got[0].keys()) == ["shape", "kernel", "ms_per_iter", "tokens_per_sec", "peak_mb"]
    assert len(got) == 4 and got[2]["shape"] == "deepseek_v2_lite" and got[3]["kernel"] == "fp8_sm100_graph"
    assert float(got[0]["tokens_per_sec"]) == 256 / 2e-3


@pytest.mark.gpu
def test_matrix_run_on_the_gpu_writes_parseable_rows(tmp_path, capsys):
    out = tmp_path / "matrix.csv"
    assert bench_cli.main(["--matrix", "--shapes", "toy_E16,mixtral_8x22B_decode", "--out", str(out), "--iters", "3",
                           "--warmup", "2"]) == 0
    with open(out) as f:
        rows = list(csv.DictReader(f))
    kernels = {(r["shape"], r["kernel"]) for r in rows}
    assert ("toy_E16", "fp8_sm100") in kernels and ("toy_E16", "fp8_sm100_graph") in kernels
    assert ("toy_E16", "fp8_sm100_block") in kernels and ("mixtral_8x22B_decode", "fp8_sm100") in kernels
    for r in rows:
        assert float(r["ms_per_iter"]) > 0 and float(r["tokens_per_sec"]) > 0 and float(r["peak_mb"]) > 0
    assert "Wrote" in capsys.readouterr().out
