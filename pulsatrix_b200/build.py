"""Builds libpsx_b200.so (the CUDA kernels and their C ABI) in-tree with nvcc for sm_100a.

    python -m pulsatrix_b200.build            # build if sources are newer than the library
    python -m pulsatrix_b200.build --force

nvcc cross-compiles, so this works on a machine without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
LIBRARY = PACKAGE / "libpsx_b200.so"
SOURCES = ["c_abi.cu", "scan_rows.cu", "merge_rows.cu", "topk_rows.cu", "shard_records.cu", "peer_exchange.cu", "no_alloc.cu", "read_floor.cu", "process_rows.cu", "row_ops.cu", "lm_head.cu", "decode_attention.cu"]
HOST_SOURCES = ["determinism.cpp", "sampler.cpp", "backend.cpp", "generation.cpp"]  # the C++ API over the C ABI
CPP_TEST = PACKAGE.parent / "tests" / "cpp" / "host_api_test"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--fmad=true",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def _profiling() -> bool:
    """PSX_B200_STAGE_CLOCKS=1 builds a second library, libpsx_b200_clocks.so, whose kernels stamp the SM
    clock at their stage boundaries (a profiling aid: it also exports psx_debug_stage_clocks and
    psx_debug_merge_clocks to read the stamps back); the Python binding loads it under the same variable."""
    return os.environ.get("PSX_B200_STAGE_CLOCKS") == "1"


def _stale() -> bool:
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    deps = (list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list((PACKAGE / "host").glob("*.cpp")) +
            list((PACKAGE.parent / "include").rglob("*.h*")))
    return any(p.stat().st_mtime > built for p in deps)


def build(force: bool = False, verbose: bool = False, defines=(), output: Path | None = None) -> Path:
    """defines / output: a variant library for experiments (e.g. defines=["PSX_STREAM_RING=4"]), written to
    `output` and loaded by pointing PSX_B200_LIBRARY at it; the default library is not touched."""
    profiling = _profiling()
    library = PACKAGE / "libpsx_b200_clocks.so" if profiling else LIBRARY
    variant = output is not None
    if variant:
        library = Path(output)
    if not force and not profiling and not variant and not _stale():
        return LIBRARY
    objects = []
    build_dir = PACKAGE / ("build_clocks" if profiling else "build_" + library.stem if variant else "build")
    build_dir.mkdir(exist_ok=True)
    procs = []
    for src in SOURCES:
        obj = build_dir / (src + ".o")
        cmd = ["nvcc", *NVCC_FLAGS, *(["-DPSX_STAGE_CLOCKS"] if profiling else []), *[f"-D{d}" for d in defines],
               *(["-Xptxas", "-v"] if verbose else []),
               "-c", str(CSRC / src), "-o", str(obj)]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objects.append(str(obj))
    include = str(PACKAGE.parent / "include")
    for src in HOST_SOURCES:
        obj = build_dir / (src + ".o")
        cmd = ["nvcc", "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-I", include,
               "-c", str(PACKAGE / "host" / src), "-o", str(obj)]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objects.append(str(obj))
    for src, proc in procs:
        out, _ = proc.communicate()
        if verbose or proc.returncode != 0:
            sys.stderr.write(out)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    subprocess.run(["nvcc", "-arch=sm_100a", "-shared", "-o", str(library), *objects, "-lcudart"], check=True)
    if not profiling and not variant:
        build_cpp_test()
    return library


def build_cpp_test() -> Path:
    """The C++ test program of the host API (tests/cpp/host_api_test.cpp), linked against the library."""
    source = CPP_TEST.with_suffix(".cpp")
    if source.exists():
        cuda = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
        subprocess.run(["g++", "-std=c++17", "-O1", "-ffp-contract=off", "-I", str(PACKAGE.parent / "include"),
                        "-I", str(cuda / "include"), str(source), "-o", str(CPP_TEST), "-L", str(PACKAGE), "-lpsx_b200",
                        "-L", str(cuda / "lib64"), "-lcudart", f"-Wl,-rpath,{PACKAGE}", "-Wl,-rpath,$ORIGIN/../../pulsatrix_b200"],
                       check=True)
    return CPP_TEST


if __name__ == "__main__":
    extra = [a[2:] for a in sys.argv[1:] if a.startswith("-D")]
    out = [a.split("=", 1)[1] for a in sys.argv[1:] if a.startswith("--output=")]
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, defines=extra, output=Path(out[0]) if out else None))
