"""Host code under AddressSanitizer + UndefinedBehaviorSanitizer: the benchmark core, the MPI
bridge, one driver, the single-host MPI subset, the ring wrapper and the int8 codec are
compiled into ONE instrumented executable and run as two ranks on the CPU. Any report
(heap overflow, use after free, misaligned access, signed overflow ...) fails the run."""
import os
import shutil
import subprocess
import uuid
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
SAN = ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined", "-fno-omit-frame-pointer", "-g", "-O1"]


def _build(tmp_path, test):
    core = [ROOT / "csrc/core" / f for f in ("cli.c", "validate.c", "oracle.c", "bindump.c", "perf.c", "devmap.c", "mpi_bridge.c")]
    metrics = sorted((ROOT / "userconfig/deviation_metric_examples").glob("*.c"))
    ex = ROOT / "userconfig/wrapper_code_examples"
    srcs = [ROOT / "csrc/bench/mpi" / f"{test}.c", *core, *metrics, ROOT / "csrc/minimpi/minimpi.c",
            ex / "communication/plain_mpi_compress/plain_mpi_compress.c", ROOT / "csrc/wrappers/mpi_compress_tools.c",
            ex / "compression/int8_block/mpi_int8_wrapper.c"]
    exe = tmp_path / f"{test}_san"
    inc = [ROOT / "include/ccb/compat", ROOT / "include", ROOT / "userconfig/deviation_metric_examples", ROOT / "csrc/minimpi",
           ROOT / "csrc/bench/mpi"]
    cmd = ["gcc", *SAN, "-Wno-format-truncation", *[f"-I{i}" for i in inc], *map(str, srcs), "-o", str(exe), "-lm", "-ldl", "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0 and ("asan" in r.stderr.lower() or "sanitize" in r.stderr.lower()):
        pytest.skip("this compiler has no sanitizer runtime")
    assert r.returncode == 0, r.stderr[-3000:]
    return exe


@pytest.mark.skipif(shutil.which("gcc") is None, reason="no gcc")
@pytest.mark.parametrize("test,args", [
    ("allreduce", ["-L", "4096,1000003", "-i", "2", "-w", "1", "-d", "float", "-v", "-t", "1e30", "-e", "mse,rel_l2,psnr,error_distrib"]),
    ("reducescatter", ["-m", "1024:65536:4", "-i", "1", "-w", "1", "-d", "float", "-v", "-t", "1e30"]),
])
def test_mpi_stack_is_clean_under_asan_and_ubsan(tmp_path, test, args):
    exe = _build(tmp_path, test)
    job = "san" + uuid.uuid4().hex[:8]
    procs = []
    for r in range(2):
        env = dict(os.environ, OMPI_COMM_WORLD_RANK=str(r), OMPI_COMM_WORLD_SIZE="2", OMPI_COMM_WORLD_LOCAL_RANK=str(r),
                   CCB_MINIMPI_JOB=job, ASAN_OPTIONS="detect_leaks=0:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1",
                   METRIC_ERROR_DISTRIB_OUTPUT=str(tmp_path / "error_distrib.txt"))
        env.pop("LD_PRELOAD", None)
        procs.append(subprocess.Popen([str(exe), *args], cwd=tmp_path, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=300) for p in procs]
    for p, (out, err) in zip(procs, outs):
        assert p.returncode == 0, out[-1500:] + err[-3000:]
        assert "ERROR: AddressSanitizer" not in err and "runtime error:" not in err, err[-3000:]
    assert "rel_l2" in outs[0][0] or test != "allreduce"
