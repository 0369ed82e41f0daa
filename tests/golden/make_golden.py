"""Generates the golden fixtures in this directory from the reference's OWN kernels.

Needs a GPU and the harness binaries oracle/_ref/ref_harness_s0,
oracle/_ref/ref_harness_s4, oracle/_ref/ref_harness_gs and oracle/_ref/ref_harness_a0 (built by `make -C oracle ref` where the reference
checkout is available; they compile the reference's .cu files in place and launch
its kernels unmodified).  Usage, on a machine with a GPU:

    python tests/golden/make_golden.py OUTDIR

writes one .npz per case into OUTDIR; the committed fixtures were produced this
way on a B200 and copied here.  Inputs are stored only for the smallest case of
each family (they pin the generator); the larger cases store outputs and are
checked against oracle-generated inputs.
"""
import os
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REF = os.path.join(ROOT, "oracle", "_ref")

S4_CASES = [(128, 256, 128, True), (64, 200, 96, True), (256, 512, 384, False), (128, 256, 1024, False)]
S0_CASES = [(64, 64, 64, True), (40, 56, 48, True), (96, 80, 160, False)]
S0_SCENARIOS = ("clean", "inject", "two_rc", "same_row", "cancel")
# GEMM + softmax cross-nonlinearity check: (M, N, K, fault_row, fault_col, fault_value)
GS_CASES = [(64, 64, 64, 32, 32, 1.0), (96, 200, 128, 5, 199, -0.75), (128, 1000, 256, 100, 0, 2.5)]
GS_PHASES = ("clean", "fault", "recovered")
# attention (the reference's scalar kernel A0): (B, H, N, D, causal, [(stage, query, index, value), ...]); batch 0, head 0
A0_CASES = [(1, 2, 256, 128, 0, [(0, 0, 0, 0.0), (1, 128, 128, 1.0), (1, 255, 3, -2.5), (2, 128, 128, 0.25), (3, 128, 128, 0.75),
                                 (4, 128, 64, 0.5), (4, 7, 127, -1.0)]),
            (1, 2, 256, 64, 1, [(0, 0, 0, 0.0), (1, 200, 100, 1.5), (4, 200, 32, 0.5), (2, 200, 100, 0.25)]),
            (2, 1, 384, 128, 1, [(0, 0, 0, 0.0), (1, 383, 0, 3.0), (4, 130, 5, 0.75)]),
            # sequence lengths that are not whole tiles
            (1, 2, 200, 128, 0, [(0, 0, 0, 0.0), (1, 199, 150, 2.0), (4, 199, 64, 0.5), (2, 130, 199, 0.25), (3, 64, 10, 0.75)]),
            (1, 2, 333, 64, 1, [(0, 0, 0, 0.0), (1, 332, 300, 1.5), (4, 260, 10, 0.5)])]


def _read(path, dtype):
    return np.fromfile(path, dtype=dtype)


def run_s4(m, n, k, keep_inputs, outdir):
    with tempfile.TemporaryDirectory() as tmp:
        subprocess.run([os.path.join(REF, "ref_harness_s4"), str(m), str(n), str(k), tmp], check=True)
        data = {name: _read(os.path.join(tmp, name + ".f32"), np.float32) for name in
                ("a_sums", "a_mags", "b_sums", "b_mags", "expected_rows", "row_scales", "expected_cols", "col_scales")}
        a = _read(os.path.join(tmp, "a.u8"), np.uint8)
        b = _read(os.path.join(tmp, "b.u8"), np.uint8)
        if keep_inputs:
            data["a"], data["b"] = a, b
        else:  # a short fingerprint instead of the bytes
            data["a_head"], data["b_head"] = a[:256], b[:256]
            data["a_sum"], data["b_sum"] = np.uint64(a.astype(np.uint64).sum()), np.uint64(b.astype(np.uint64).sum())
        data["shape"] = np.array([m, n, k], dtype=np.int32)
        np.savez_compressed(os.path.join(outdir, f"s4_prepare_{m}x{n}x{k}.npz"), **data)


def run_s0(m, n, k, keep_inputs, outdir):
    with tempfile.TemporaryDirectory() as tmp:
        subprocess.run([os.path.join(REF, "ref_harness_s0"), str(m), str(n), str(k), tmp], check=True)
        data = {name: _read(os.path.join(tmp, name + ".f32"), np.float32) for name in
                ("c_gemm", "expected_rows", "expected_cols", "row_scales", "col_scales")}
        for s in S0_SCENARIOS:
            data["c_" + s] = _read(os.path.join(tmp, f"c_{s}.f32"), np.float32)
            data["counters_" + s] = _read(os.path.join(tmp, f"counters_{s}.i32"), np.int32)
        if keep_inputs:
            data["a"] = _read(os.path.join(tmp, "a.u8"), np.uint8)
            data["b"] = _read(os.path.join(tmp, "b.u8"), np.uint8)
        data["shape"] = np.array([m, n, k], dtype=np.int32)
        np.savez_compressed(os.path.join(outdir, f"s0_path_{m}x{n}x{k}.npz"), **data)


def run_gs(m, n, k, fault_row, fault_col, fault_value, outdir):
    with tempfile.TemporaryDirectory() as tmp:
        subprocess.run([os.path.join(REF, "ref_harness_gs"), str(m), str(n), str(k), str(fault_row), str(fault_col), str(fault_value),
                        tmp], check=True)
        data = {"a": _read(os.path.join(tmp, "a.u8"), np.uint8), "b": _read(os.path.join(tmp, "b.u8"), np.uint8),
                "logits": _read(os.path.join(tmp, "logits.f32"), np.float32),
                "expected_sum": _read(os.path.join(tmp, "expected_sum.f64"), np.float64),
                "expected_weighted": _read(os.path.join(tmp, "expected_weighted.f64"), np.float64)}
        for p in GS_PHASES:
            prob = _read(os.path.join(tmp, f"probabilities_{p}.f32"), np.float32)
            if m * n <= 20000:
                data["probabilities_" + p] = prob
            else:  # the large case keeps the faulty row only
                data["probabilities_row_" + p] = prob.reshape(m, n)[fault_row].copy()
            for name in ("actual_sum", "actual_weighted", "probability_sum", "log_z", "correction_delta"):
                data[f"{name}_{p}"] = _read(os.path.join(tmp, f"{name}_{p}.f64"), np.float64)
            for name in ("detected", "estimated_col", "counts"):
                data[f"{name}_{p}"] = _read(os.path.join(tmp, f"{name}_{p}.i32"), np.int32)
        data["shape"] = np.array([m, n, k], dtype=np.int32)
        data["fault"] = np.array([fault_row, fault_col, fault_value], dtype=np.float64)
        np.savez_compressed(os.path.join(outdir, f"gs_{m}x{n}x{k}.npz"), **data)


def run_a0(batch, heads, seq, dim, causal, scenarios, outdir):
    with tempfile.TemporaryDirectory() as tmp:
        args = [os.path.join(REF, "ref_harness_a0"), str(batch), str(heads), str(seq), str(dim), str(causal), tmp]
        args += [f"{s}:{q}:{i}:{v}" for s, q, i, v in scenarios]
        subprocess.run(args, check=True)
        data = {name: _read(os.path.join(tmp, name + ".u8"), np.uint8) for name in ("q", "k", "v")}
        clean = None
        for n, (stage, query, _, _) in enumerate(scenarios):
            out = _read(os.path.join(tmp, f"out_{n}.f32"), np.float32).reshape(batch, heads, seq, dim)
            if stage == 0:  # the clean output in full; of a fault scenario the faulty query's row and how far all other rows moved
                clean = out
                data[f"out_{n}"] = out.ravel().astype(np.float16)  # |O| < 1: 5e-4 absolute, well inside the 2e-3 of the comparison
            else:
                data[f"row_{n}"] = out[0, 0, query].copy()
                rest = np.abs(out - clean)
                rest[0, 0, query] = 0.0
                data[f"others_{n}"] = np.float32(rest.max())
            data[f"stats_{n}"] = _read(os.path.join(tmp, f"stats_{n}.i32"), np.int32)
        data["shape"] = np.array([batch, heads, seq, dim, causal], dtype=np.int32)
        data["scenarios"] = np.array(scenarios, dtype=np.float64)
        np.savez_compressed(os.path.join(outdir, f"a0_{batch}x{heads}x{seq}x{dim}_c{causal}.npz"), **data)


def main():
    outdir = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "golden_out")
    only = sys.argv[2].split(",") if len(sys.argv) > 2 else ["s4", "s0", "gs", "a0"]  # optional: which families to regenerate
    os.makedirs(outdir, exist_ok=True)
    for family, cases, run in (("s4", S4_CASES, run_s4), ("s0", S0_CASES, run_s0), ("gs", GS_CASES, run_gs), ("a0", A0_CASES, run_a0)):
        if family in only:
            for case in cases:
                run(*case, outdir)
    print("golden fixtures written to", outdir, sorted(os.listdir(outdir)))


if __name__ == "__main__":
    main()
