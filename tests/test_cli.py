"""The MergePathSpMM command-line program: the reference's argv contract
(src/MergePathSpMM.cu:114-124,141)."""
import os
import subprocess

import pytest

import cases

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CLI = os.path.join(ROOT, "mergepath-spmm_b200", "lib", "MergePathSpMM")


@pytest.fixture(scope="module")
def cli(mps):
    from mergepath_spmm_b200 import build
    return build.build_cli()


@pytest.fixture(scope="module")
def c1_file(tmp_path_factory, mps):
    rp, col = cases.c1_rmat()
    p = str(tmp_path_factory.mktemp("cli") / "c1.csr")
    mps.save_csr(p, rp, col)
    return p, len(rp) - 1, len(col)


def test_too_few_arguments_prints_the_reference_usage_and_exits_minus_one(cli):
    r = subprocess.run([cli, "graph.csr", "16", "8"], capture_output=True, text=True)
    assert r.returncode == 255  # exit(-1)
    assert r.stdout.strip() == "Usage: ./application <input_file> <dimension> <cost> <threads_per_warp> <repeat>"


def test_missing_file_is_an_error(cli):
    r = subprocess.run([cli, "/nonexistent/graph.csr", "16", "8", "2", "1"], capture_output=True, text=True)
    assert r.returncode == 1 and "cannot open" in r.stderr


def test_first_line_matches_the_reference(cli, c1_file):
    path, n, nnz = c1_file
    r = subprocess.run([cli, path, "16", "8", "32", "1"], capture_output=True, text=True)
    assert r.stdout.splitlines()[0] == f"Total number of rows: {n} and non-zeros: {nnz}"
    assert "threads_per_warp 32 exceeds" in r.stderr  # clamped where the reference exits


def test_binary_sidecar_is_accepted_in_place_of_the_text_file(cli, c1_file, tmp_path, mps):
    path, n, nnz = c1_file
    rp, col = cases.c1_rmat()
    side = str(tmp_path / "c1.bin")
    mps.save_csr_bin(side, rp, col)
    r = subprocess.run([cli, side, "16", "8", "1", "1"], capture_output=True, text=True)
    assert r.stdout.splitlines()[0] == f"Total number of rows: {n} and non-zeros: {nnz}"


def test_any_cost_the_reference_accepts_is_accepted(cli, c1_file):
    """The reference's command line takes any positive cost (src/MergePathSpMM.cu:121); so does this one - without a
    device the run stops at the device, not at the cost."""
    path, n, nnz = c1_file
    for cost in ("1000", "100000000"):
        r = subprocess.run([cli, path, "16", cost, "1", "1"], capture_output=True, text=True)
        assert "shared memory" not in r.stderr and r.stdout.startswith("Total number of rows")


@pytest.mark.gpu
@pytest.mark.parametrize("extra", [[], ["--values=gcn"], ["--dtype=f16", "--values=gcn"]])
def test_runs_and_checks_on_the_gpu(cli, c1_file, cuda, extra):
    path, n, nnz = c1_file
    for dim in ("16", "64"):
        r = subprocess.run([cli, path, dim, "8", "2", "3", "--check"] + extra, capture_output=True, text=True)
        assert r.returncode == 0, r.stdout + r.stderr
        assert "check: 0 elements outside tolerance" in r.stdout and "GFLOP/s" in r.stdout
    r = subprocess.run([cli, path, "64", "100000", "1", "2", "--check"] + extra, capture_output=True, text=True)   # a cost far beyond one tile
    assert r.returncode == 0 and "check: 0 elements outside tolerance" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_fp16_twin_program_defaults_to_fp16_storage(cli, c1_file, cuda):
    """MergePathSpMM_fp16: the reference's second program (src/MergePathSpMM_fp16.cu:111-125), same argv."""
    path, n, nnz = c1_file
    r = subprocess.run([cli + "_fp16", path, "32", "8", "1", "2", "--check", "--values=gcn"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "dtype: f16" in r.stdout and "check: 0 elements outside tolerance" in r.stdout
    r = subprocess.run([cli + "_fp16", path, "32", "8"], capture_output=True, text=True)
    assert r.returncode == 255


@pytest.mark.gpu
def test_multi_gpu_with_nccl_gather(cli, c1_file, cuda):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two devices")
    path, n, nnz = c1_file
    r = subprocess.run([cli, path, "32", "8", "1", "3", "--values=gcn", "--gpus=2", "--gather-c", "--check"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "check: 0 elements outside tolerance" in r.stdout and "all-gather of C over NCCL" in r.stdout
