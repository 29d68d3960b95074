"""C++ stage checker of the MoE layer (rf_moe_stage_check.cu): build helper."""
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCE = os.path.join(HERE, "rf_moe_stage_check.cu")
BINARY = os.path.join(HERE, "rf_moe_stage_check")


def build(force: bool = False) -> str:
    """Compiles the checker next to its source (host code only; nvcc provides cuda_fp16.h and cudart)."""
    header = os.path.join(os.path.dirname(os.path.dirname(HERE)), "include", "rf_b200.h")
    if not force and os.path.exists(BINARY) and all(
            os.path.getmtime(BINARY) >= os.path.getmtime(p) for p in (SOURCE, header)):
        return BINARY
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler",
           "-fopenmp,-ffp-contract=off", "-o", BINARY, SOURCE, "-ldl"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building rf_moe_stage_check:\n" + res.stdout + res.stderr)
    return BINARY
