"""Host logic of the shape-sweep harness (mxblas_b200/bench_all.py): shape table, problem sizes per scaling
pattern and the CSV schema of the reference's bench/bench_all.py:176."""

from mxblas_b200 import bench_all as ba


def test_csv_schema_matches_the_reference_header():
    assert ba.CSV_HEAD == "Model,M,N,K,SM,SN,SK,Q,QN,SP,Method,Time(ms),TFLOPS,Bandwidth(GB/s)\n"
    row = ba.csv_row("llama-3-8b", 128, 6144, 4096, 1, 128, 128, False, 16, ba.SP.GB, ba.Method.MXBLAS_B200, 0.01234, 86.957, 403.4)
    assert row == "llama-3-8b,128,6144,4096,1,128,128,False,16,GB,MXBLAS_B200,0.0123,86.96,403.40\n"
    assert len(row.strip().split(",")) == len(ba.CSV_HEAD.strip().split(","))


def test_problem_sizes_per_scaling_pattern():
    assert ba.gen_problem_size(4096, 7168, 7168, ba.SP.TT) == (4096, 7168, 7168, 4096, 7168, 7168)
    assert ba.gen_problem_size(4096, 7168, 7168, ba.SP.CC) == (4096, 7168, 7168, 1, 1, 7168)
    assert ba.gen_problem_size(4096, 7168, 7168, ba.SP.GB) == (4096, 7168, 7168, 1, 128, 128)
    assert ba.gen_problem_size(4096, 7168, 7168, ba.SP.BB) == (4096, 7168, 7168, 128, 128, 128)
    assert ba.gen_problem_size(64, 7168, 7168, ba.SP.BB)[3] == 64  # a block never exceeds M


def test_shape_table_is_usable_by_every_pattern():
    shapes = ba.gemm_shapes([128, 1024])
    assert set(shapes) == set(ba.MODEL_NAMES)
    for model, lst in shapes.items():
        assert len(lst) == 2 * len(ba.GEMM_SHAPES[model])
        for m, n, k in lst:
            assert k % 128 == 0 and n % 128 == 0, (model, n, k)  # 128 x 128 blocks divide every layer


def test_rates():
    ms, tflops, gbs = ba.rates(1024, 1024, 1024, 1e-3)
    assert ms == 1.0
    assert abs(tflops - 2 * 1024**3 / 1e-3 / 1e12) < 1e-9
    assert abs(gbs - (1024 * 1024 * 2 + 2 * 1024 * 1024) / 1e-3 / 1e9) < 1e-9


def test_sweep_summary_table(tmp_path):
    """The summary of a sweep CSV: medians per pattern and M, ratio to cuBLASLt, time relative to TT."""
    import pandas as pd

    from mxblas_b200 import bench_all, plot_box

    path = tmp_path / "sweep.csv"
    rows = [bench_all.CSV_HEAD]
    for n, tf_ours, tf_lt in ((4096, 2000.0, 2500.0), (8192, 3000.0, 2800.0)):
        ms = 2.0 * 1024 * n * 4096 / tf_ours / 1e9
        rows.append(bench_all.csv_row("m", 1024, n, 4096, 1024, n, 4096, False, 16, "TT", "MXBLAS_B200", ms, tf_ours, 1.0))
        rows.append(bench_all.csv_row("m", 1024, n, 4096, 1024, n, 4096, False, 16, "TT", "CUBLASLT", ms, tf_lt, 1.0))
        rows.append(bench_all.csv_row("m", 1024, n, 4096, 1, 128, 128, False, 16, "GB", "MXBLAS_B200", 1.5 * ms, tf_ours / 1.5, 1.0))
    path.write_text("".join(rows))
    text = plot_box.summary_table(pd.read_csv(path))
    tt = [line for line in text.splitlines() if line.startswith("| TT | 1024 |")][0]
    assert "2500 (2000 .. 3000)" in tt and "| 2650 |" in tt and "| 0.94 |" in tt
    gb = [line for line in text.splitlines() if line.startswith("| GB | 1024 |")][0]
    assert "1.50x" in gb and "| - | - |" in gb
