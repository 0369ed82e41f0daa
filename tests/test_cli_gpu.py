"""The per-stage command-line programs on a GPU: same flags, `key: value` report and
exit-code rule as the reference's programs (which are their own tests: each one
verifies itself and returns 0 or 1, src/s4_cluster_multicast_abft_fp8_gemm.cu:723-726, 784)."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BUILD = os.path.join(ROOT, "build")


def run(program, *args):
    exe = os.path.join(BUILD, program)
    if not os.path.exists(exe):
        subprocess.run(["make", "-C", ROOT, "cli"], check=True, stdout=subprocess.DEVNULL)
    out = subprocess.run([exe, *map(str, args)], capture_output=True, text=True, timeout=600)
    report = {}
    for line in out.stdout.splitlines():
        key, sep, value = line.partition(": ")
        if sep:
            report.setdefault(key, value)
    return out.returncode, report, out.stderr


def test_stage_program_clean_and_injected():
    rc, rep, _ = run("stage_abft_fp8_gemm", "--m", 1024, "--n", 1024, "--k", 1024, "--warmup", 1, "--repeat", 3)
    assert rc == 0 and rep["verification"] == "PASS"
    assert rep["shape"].startswith("M=1024 N=1024 K=1024, abft_tiles=256")
    assert (rep["bad_tiles"], rep["corrected_tiles"]) == ("0", "0")
    for key in ("metadata_cache_bytes", "input_metadata_time_ms", "expected_metadata_time_ms", "metadata_prepare_time_ms",
                "first_fused_gemm_abft_time_ms", "first_call_total_ms", "first_call_tflops", "avg_fused_gemm_abft_time_ms",
                "amortized_time_ms", "amortized_tflops", "fused_gemm_tflops", "abft_tolerance", "verification_samples",
                "sampled_max_absolute_error", "sampled_max_tolerance_ratio", "layout"):
        assert key in rep, key
    assert rep["layout"] == "A=[M,K] row-major, B=[N,K] column-major, C=[N,M] column-major"
    assert float(rep["sampled_max_tolerance_ratio"]) <= 1.0 and rep["verification_samples"] == "64"
    # `--name=value` grammar and the deterministic fault of the reference (s4:449-453)
    rc, rep, _ = run("stage_abft_fp8_gemm", "--m=512", "--n=512", "--k=256", "--repeat=2", "--inject-fault", "--fault-value", 2.5)
    assert rc == 0 and (rep["bad_tiles"], rep["corrected_tiles"], rep["verification"]) == ("1", "1", "PASS")
    # one-CTA form (M not a multiple of 256) and a fault below the threshold: the run fails like the reference's would
    rc, rep, _ = run("stage_abft_fp8_gemm", "--m", 384, "--n", 256, "--k", 128, "--repeat", 1, "--inject-fault", "--fault-value", 1e-4)
    assert rc == 1 and rep["bad_tiles"] == "0" and rep["verification"] == "FAIL"


def test_stage_program_added_flags():
    """--fault2 (the tile is reported, not corrected), --seed, --json, --gpus."""
    import json
    rc, rep, _ = run("stage_abft_fp8_gemm", "--m", 512, "--n", 512, "--k", 256, "--repeat", 2, "--fault2", "--fault-value", 3.0)
    assert rc == 0 and (rep["bad_tiles"], rep["corrected_tiles"], rep["multi_fault_tiles"], rep["verification"]) == ("1", "0", "1", "PASS")
    exe = os.path.join(BUILD, "stage_abft_fp8_gemm")
    out = subprocess.run([exe, "--m", "256", "--n", "256", "--k", "128", "--repeat", "2", "--seed", "7", "--json"], capture_output=True,
                         text=True, timeout=300)
    assert out.returncode == 0
    doc = json.loads(out.stdout.splitlines()[-1])
    assert doc["verification"] == "PASS" and doc["bad_tiles"] == 0 and doc["gpus"] == 1 and doc["fused_gemm_tflops"] > 0
    rc, rep, err = run("stage_abft_fp8_gemm", "--gpus", 64)
    assert rc == 1 and "needs that many devices" in err
    import torch
    if torch.cuda.device_count() >= 2:
        rc, rep, _ = run("stage_abft_fp8_gemm", "--m", 1024, "--n", 512, "--k", 256, "--repeat", 2, "--gpus", 2, "--inject-fault")
        assert rc == 0 and (rep["gpus"], rep["rows_per_gpu"], rep["bad_tiles"], rep["corrected_tiles"]) == ("2", "512", "1", "1")
        # the record came through the all-gather with the tile id of the whole product: tile 64 = tile row 8, the first of GPU 1
        assert rep["report_gather"].startswith("ncclAllGather") and rep["fault_record_0"].startswith("tile=64 gpu=1 bad_rows=1 bad_cols=1 row=32 col=32")


def test_stage_program_rejects_bad_shapes():
    for args in (["--m", 0], ["--n", 0], ["--k", -8], ["--repeat", 0]):
        rc, rep, err = run("stage_abft_fp8_gemm", *args)
        assert rc == 1 and not rep and "Invalid options" in err
    # boundary tiles: any M, N and K
    rc, rep, _ = run("stage_abft_fp8_gemm", "--m", 256, "--n", 200, "--k", 96, "--repeat", 2, "--inject-fault", "--fault-value", 3.0)
    assert rc == 0 and (rep["bad_tiles"], rep["corrected_tiles"], rep["verification"]) == ("1", "1", "PASS")
    assert rep["shape"].startswith("M=256 N=200 K=96, abft_tiles=16")
    rc, rep, _ = run("stage_abft_fp8_gemm", "--m", 100, "--n", 300, "--k", 50, "--repeat", 2, "--inject-fault", "--fault-value", 3.0)
    assert rc == 0 and (rep["bad_tiles"], rep["corrected_tiles"], rep["verification"]) == ("1", "1", "PASS")


def test_campaign_program():
    rc, rep, _ = run("fault_campaign", "--m", 1024, "--n", 1024, "--k", 1024, "--warmup", 1, "--repeat", 1, "--fault-trials", 60,
                     "--fault-seed", 12345, "--double-trials", 10)
    assert rc == 0 and rep["verification"] == "PASS"
    assert rep["fault_campaign_trials"] == "60" and rep["fault_campaign_seed"] == "12345"
    # uniform(-1,1) inputs at K=1024: threshold ~0.34, every fault of magnitude >= 1 is caught
    assert rep["fault_campaign_detected"] == "60" and rep["fault_campaign_corrected"] == "60"
    assert rep["fault_campaign_missed"] == "0" and rep["fault_campaign_miscorrected"] == "0"
    assert rep["fault_campaign_correction_rate_percent"] == "100.000"
    assert rep["double_fault_reported_uncorrected"] == "10" and rep["double_fault_silently_corrected"] == "0"
    assert sum(int(rep[f"fault_campaign_bin_{i}"].split("trials=")[1].split()[0]) for i in range(4)) == 60


def test_attention_program():
    rc, rep, _ = run("ft_flash_attention", "--batch", 1, "--heads", 2, "--sequence", 512, "--repeat", 2)
    assert rc == 0 and rep["verification"] == "PASS" and rep["mismatches"] == "0"
    assert (rep["score_detected"], rep["pv_detected"], rep["failed_rows"]) == ("0", "0", "0")
    rc, rep, _ = run("ft_flash_attention", "--batch", 1, "--heads", 2, "--sequence", 512, "--repeat", 1, "--fault-stage", "score",
                     "--fault-value", 4.0)
    assert rc == 0 and (rep["score_detected"], rep["score_corrected"]) == ("1", "1")
    assert rep["fault_target"].startswith("batch=0 head=0 query=256 index=256")  # defaults of a0:193-199
    rc, rep, _ = run("ft_flash_attention", "--batch", 1, "--heads", 2, "--sequence", 512, "--repeat", 1, "--fault-stage=output",
                     "--fault-value", 0.5, "--dist", "grid")
    assert rc == 0 and (rep["pv_detected"], rep["pv_corrected"], rep["failed_rows"]) == ("1", "1", "0")
    rc, rep, _ = run("ft_flash_attention", "--batch", 1, "--heads", 2, "--sequence", 512, "--repeat", 1, "--causal", "--fault-stage",
                     "score", "--fault-value", 4.0)
    assert rc == 0 and rep["shape"].endswith("causal=1") and (rep["score_detected"], rep["score_corrected"]) == ("1", "1")
    assert rep["fault_target"].startswith("batch=0 head=0 query=256 index=128")  # causal default of a14:261
    # two faults in one score tile: not locatable, the tile is replayed on the CUDA cores and the output verifies
    rc, rep, _ = run("ft_flash_attention", "--batch", 1, "--heads", 2, "--sequence", 512, "--repeat", 1, "--fault-stage", "score",
                     "--fault-value", 4.0, "--fault2-query", 260, "--fault2-index", 300, "--fault2-value", -3.0)
    assert rc == 0 and (rep["score_detected"], rep["score_corrected"], rep["score_replayed"], rep["score_uncorrected"]) == ("1", "0", "1", "0")
    rc, _, err = run("ft_flash_attention", "--sequence", 256, "--causal", "--fault-stage", "score", "--fault-query", 10, "--fault-index", 20)
    assert rc == 1 and "must not exceed" in err
    rc, rep, _ = run("ft_flash_attention", "--batch", 1, "--heads", 2, "--sequence", 512, "--head-dim", 64, "--repeat", 1, "--fault-stage",
                     "output", "--fault-value", 0.5)  # the reference's default head dimension (a14:114)
    assert rc == 0 and rep["shape"].startswith("B=1 H=2 N=512 D=64") and (rep["pv_detected"], rep["pv_corrected"]) == ("1", "1")
    rc, _, err = run("ft_flash_attention", "--head-dim", 96)
    assert rc == 1 and "Invalid options" in err


def test_gemm_softmax_program():
    """Same lines and exit-code rule as the reference's prototype (src/gemm_softmax_abft.cu:465-521)."""
    exe = os.path.join(BUILD, "gemm_softmax_abft")
    if not os.path.exists(exe):
        subprocess.run(["make", "-C", ROOT, "cli"], check=True, stdout=subprocess.DEVNULL)
    out = subprocess.run([exe], capture_output=True, text=True, timeout=300)  # defaults: 64^3, fault +1 at (32, 32)
    assert out.returncode == 0
    lines = out.stdout.splitlines()
    assert lines[0] == "GEMM + Softmax cross-nonlinearity ABFT"
    assert lines[1] == "shape: M=64 N=64 K=64, scale=1/sqrt(K), input=FP8 E4M3, output=FP32"
    assert any(line.startswith("clean run: detected_rows=0 located_rows=0 max_projection_residual=") for line in lines)
    assert "fault: row=32 col=32 injected_delta=+1.000000" in lines
    assert "detection: detected_rows=1 located_rows=1 estimated_col=32 estimated_delta=+1.000000" in lines
    assert any(line.startswith("recovery: post_detected_rows=0 max_probability_error=") for line in lines)
    assert lines[-1] == "verification: PASS"
    out = subprocess.run([exe, "--m", "100", "--n", "300", "--k", "72", "--fault-row", "99", "--fault-col", "0", "--fault-value", "-2.5"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "estimated_col=0 estimated_delta=-2.500000" in out.stdout
    out = subprocess.run([exe, "--no-fault", "--m", "256", "--n", "512", "--k", "128"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "fault:" not in out.stdout
    out = subprocess.run([exe, "--n", "1"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 1 and "Invalid shape, fault, or tolerance option." in out.stderr
    out = subprocess.run([exe, "--fault-row", "64"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 1 and "Fault position must satisfy row < M and col < N." in out.stderr


def test_cublaslt_program():
    rc, rep, _ = run("cublaslt_fp8_bench", "--m", 1024, "--n", 1024, "--k", 1024, "--warmup", 2, "--repeat", 5)
    assert rc == 0 and rep["verification"] == "PASS" and rep["benchmark"] == "cuBLASLt FP8 E4M3 GEMM"
    assert float(rep["throughput_tflops"]) > 0 and int(rep["heuristic_algorithms"]) >= 1
