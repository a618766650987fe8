"""Failure handling of the data-parallel exchange, driven from the host: a stand-in communicator library (built here from
the C source below and selected with OM_NCCL_LIBRARY) reports an asynchronous error, or delays a reduction for a bounded
time, on demand. No GPU faults, traps or hangs: the error is an error code, the delay is a sleep of a few hundred
milliseconds in a host callback on the communication stream. Each case runs in its own process, because the library binds
its communicator once per process."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)

STUB = r'''
#include <cuda_runtime.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>
typedef struct { char internal[128]; } ncclUniqueId;
typedef void* ncclComm_t;
typedef int ncclResult_t;   /* 0 success, 1 unhandled cuda error, 2 system error, 7 in progress */
static int g_comm;
int ncclGetUniqueId(ncclUniqueId* id) { memset(id, 7, sizeof *id); return 0; }
int ncclCommInitRank(ncclComm_t* comm, int n, ncclUniqueId id, int rank) { (void)n; (void)id; (void)rank; *comm = &g_comm; return 0; }
int ncclCommDestroy(ncclComm_t c) { (void)c; return 0; }
int ncclCommAbort(ncclComm_t c) { (void)c; return 0; }
int ncclCommGetAsyncError(ncclComm_t c, int* e) { (void)c; const char* s = getenv("STUB_ASYNC_ERROR"); *e = s ? atoi(s) : 0; return 0; }
static void CUDART_CB nap(void* p) { (void)p; const char* s = getenv("STUB_DELAY_MS"); usleep((s ? atoi(s) : 0) * 1000); }
int ncclAllReduce(const void* a, void* b, size_t n, int t, int op, ncclComm_t c, cudaStream_t s) {
  (void)a; (void)b; (void)n; (void)t; (void)op; (void)c;
  if (getenv("STUB_DELAY_MS")) return cudaLaunchHostFunc(s, nap, 0) == cudaSuccess ? 0 : 1;   /* a rank of one: the sum is the input */
  return 0;
}
const char* ncclGetErrorString(int r) { return r == 2 ? "stand-in: system error" : "stand-in: error"; }
'''

CASE = r'''
import os, sys, time, ctypes as C
import numpy as np
sys.path.insert(0, os.path.join(%(root)r, "onemodel-csharp_b200"))
import om_binding as omb
from om_binding import i32, i64
ctx = omb.Context(0, 0)
buf = (C.c_uint8 * 128)()
ctx.call("om_dp_unique_id", ctx.handle, buf)
ctx.call("om_dp_init", ctx.handle, buf, i32(0), i32(1))
g = ctx.to_device(np.ones(1024, np.float32))
ctx.call("om_dp_register_bucket", ctx.handle, i32(0), g.ptr, i64(1024))
ctx.call("om_dp_allreduce_bucket", ctx.handle, i32(0))
mode = sys.argv[1]
t0 = time.perf_counter()
try:
    ctx.call("om_dp_wait", ctx.handle, i32(50))
    print("RESULT ok")
except omb.OmError as e:
    print("RESULT", e.status, str(e).replace("\n", " "))
print("WAITED_MS", int((time.perf_counter() - t0) * 1000))
try:
    ctx.call("om_dp_allreduce_bucket", ctx.handle, i32(0))
    print("AGAIN ok")
except omb.OmError as e:
    print("AGAIN", e.status, str(e).replace("\n", " "))
time.sleep(0.5)          # a delayed reduction has finished by now
ctx.sync()               # the context itself is intact: its stream drains and an ordinary kernel runs
out = ctx.zeros((8,))
ctx.call("om_fill", ctx.handle, out.ptr, C.c_float(3.0), i64(8))
ctx.sync()
print("USABLE", bool(np.all(out.numpy() == 3.0)))
ctx.close()
'''


@pytest.fixture(scope="module")
def stub(tmp_path_factory):
    d = tmp_path_factory.mktemp("stub")
    src, lib = d / "stub_nccl.c", d / "libstub_nccl.so"
    src.write_text(STUB)
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    subprocess.check_call(["gcc", "-shared", "-fPIC", "-O1", "-o", str(lib), str(src), f"-I{cuda}/include", f"-L{cuda}/lib64", "-lcudart",
                           f"-Wl,-rpath,{cuda}/lib64"])
    return str(lib)


def run_case(tmp_path, stub, mode, **env):
    script = tmp_path / "case.py"
    script.write_text(CASE % {"root": ROOT})
    e = dict(os.environ, OM_NCCL_LIBRARY=stub, **env)
    p = subprocess.run([sys.executable, str(script), mode], env=e, capture_output=True, text=True, timeout=240)
    assert p.returncode == 0, p.stderr[-3000:]
    return dict(line.split(" ", 1) for line in p.stdout.strip().splitlines())


def test_exchange_without_faults_completes(tmp_path, stub):
    r = run_case(tmp_path, stub, "plain")
    assert r["RESULT"] == "ok" and r["AGAIN"] == "ok" and r["USABLE"] == "True"


def test_asynchronous_communicator_error_is_reported_and_the_group_refuses_further_work(tmp_path, stub):
    """ncclCommGetAsyncError reports a system error: om_dp_wait returns OM_ERR_NCCL and aborts the communicator; the next
    reduction is refused with OM_ERR_NCCL instead of being handed a dead communicator; the context stays usable."""
    r = run_case(tmp_path, stub, "async", STUB_ASYNC_ERROR="2")
    assert r["RESULT"].startswith("5 ") and "asynchronous NCCL error" in r["RESULT"]
    assert r["AGAIN"].startswith("5 ") and "aborted" in r["AGAIN"]
    assert r["USABLE"] == "True"


def test_exchange_that_overruns_the_host_deadline_times_out(tmp_path, stub):
    """The reduction takes 300 ms (a peer that is slow or gone), the deadline is 50 ms: om_dp_wait gives up with
    OM_ERR_TIMEOUT after about the deadline instead of blocking, aborts the communicator, and the context is usable once
    the stream has drained."""
    r = run_case(tmp_path, stub, "slow", STUB_DELAY_MS="300")
    assert r["RESULT"].startswith("6 ") and "not finished after 50 ms" in r["RESULT"]
    assert 40 <= int(r["WAITED_MS"]) < 250
    assert r["AGAIN"].startswith("5 ")
    assert r["USABLE"] == "True"
