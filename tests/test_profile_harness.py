"""The profiling harness keeps the reference harness's contract: option meaning, driver command lines and CSV
names (ncu_profile.py:32-122, file_name_server.py:6-45), so its CSVs can sit beside the reference's."""
import os

from vectorsparse_b200 import profile

BM = "/raid/datasets/dlmc/rn50/random_pruning/0.8/bottleneck_2_block_group3_5_1.smtx"
STEM = "dlmc/rn50/random_pruning/0.8/bottleneck_2_block_group3_5_1"


def test_csv_names_follow_the_reference_layout():
    assert profile.csv_name(BM, 256, 8, "wmma", True, "spmm") == f"./csv/spmm/{STEM}_wmma_half_sort_k256_v8.csv"
    assert profile.csv_name(BM, 64, 4, "cuda", False, "spmm", precision="single") == f"./csv/spmm/{STEM}_cuda_single_k64_v4.csv"
    assert profile.csv_name(BM, 256, 2, "wmma", True, "sddmm", "mma_shfl") == f"./csv/sddmm/{STEM}_wmma_half_sort_mma_shfl_k256_v2.csv"
    assert profile.csv_name(BM, 256, 2, "cuda", True, "sddmm", "mma_shfl") == f"./csv/sddmm/{STEM}_cuda_half_sort_k256_v2.csv"
    assert profile.csv_name(BM, 256, 8, "bell", True, "spmm", mem=True) == f"./csv/mem/spmm/{STEM}_blocked_ell_half_sort_k256_v8.csv"
    assert profile.csv_name(BM, 256, 8, None, False, "spmm") == f"./csv/spmm/{STEM}_dense_half_k256_v8.csv"
    # a synthetic pattern spec becomes one file name
    name = profile.csv_name("synthetic:beta:256x512:s=0.9", 256, 8, "wmma", True, "spmm")
    assert name == "./csv/spmm/synthetic_beta_256x512_s0.9_wmma_half_sort_k256_v8.csv"


def test_driver_command_lines():
    spmm = profile.driver_command(BM, 256, 8, "wmma", True, True, "spmm", driver_dir=".")
    assert spmm == ["./spmm_benchmark", BM, "256", "8", "0", "1", "1", "1", "1"]
    cuda = profile.driver_command(BM, 128, 1, "cuda", False, False, "spmm", precision="single", driver_dir=".")
    assert cuda == ["./spmm_benchmark", BM, "128", "1", "1", "0", "0", "1", "0"]
    bell = profile.driver_command(BM, 128, 4, "bell", True, False, "spmm", driver_dir=".")
    assert bell[4:] == ["0", "1", "0", "2", "1"]
    sddmm = profile.driver_command(BM, 256, 4, "wmma", True, False, "sddmm", "mma_shfl", driver_dir=".")
    assert sddmm == ["./sddmm_benchmark", BM, "256", "4", "0", "2", "1", "0", "1", "1"]


def test_profiler_command_keeps_clocks_alone_and_the_reference_flags():
    cmd = profile.profile_command("ncu", "out.csv", ["./spmm_benchmark", "x"], mem=True)
    joined = " ".join(cmd)
    assert "--clock-control none" in joined
    for flag in ("-f", "--csv", "--cache-control all", "--profile-from-start 0", "--log-file out.csv",
                 "--metrics l1tex__m_xbar2l1tex_read_bytes_mem_lg_op_ld.sum"):
        assert flag in joined
    assert cmd[-2:] == ["./spmm_benchmark", "x"]


def test_duration_is_the_sum_over_kernels(tmp_path):
    f = tmp_path / "p.csv"
    f.write_text(
        "==PROF== Connected to process 1\n"
        '"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size","Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"\n'
        '"0","1","d","h","plan","1","7","(256, 1, 1)","(48, 1, 1)","0","10.0","GPU Speed Of Light Throughput","Duration","usecond","11.50"\n'
        '"0","1","d","h","plan","1","7","(256, 1, 1)","(48, 1, 1)","0","10.0","GPU Speed Of Light Throughput","Elapsed Cycles","cycle","20,000"\n'
        '"1","1","d","h","dense","1","7","(192, 1, 1)","(148, 1, 1)","0","10.0","GPU Speed Of Light Throughput","Duration","msecond","0.2"\n'
        '"2","1","d","h","gather","1","7","(192, 1, 1)","(296, 1, 1)","0","10.0","GPU Speed Of Light Throughput","Duration","nsecond","3,500"\n')
    assert abs(profile.duration_ms(str(f)) - (0.0115 + 0.2 + 0.0035)) < 1e-12
    g = tmp_path / "empty.csv"
    g.write_text("==PROF== nothing\n")
    assert profile.duration_ms(str(g)) is None


def test_dry_run_prints_the_command(capsys):
    rc = profile.main(["--bm", "synthetic:beta:64x64:s=0.9", "-k", "64", "-v", "8", "--kernel", "wmma", "--sort",
                       "--job", "spmm", "--precision", "half", "--dry"])
    assert rc == 0
    out = capsys.readouterr().out.strip()
    assert out.endswith("spmm_benchmark synthetic:beta:64x64:s=0.9 64 8 0 1 0 1 1")
    assert os.path.basename(out.split()[0]) == "spmm_benchmark"
