"""Failures of the multi-GPU plumbing, made on the host: the NCCL library cannot be opened, lacks a symbol, or its
calls return an error.  b200wmma_mg_* must answer B200WMMA_ERR_UNSUPPORTED with a message that names the cause, and
leave no handle behind.  The failing NCCL is a stand-in library built here with gcc and selected through
B200WMMA_NCCL_LIBRARY (read once per process, hence the child processes); no GPU is faulted, hung or even needed,
except for the one case that has to get past the library's "is a device current" check."""
import os
import subprocess
import sys
import textwrap

import pytest

from rocwmma_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

FAKE_NCCL = r"""
#include <stddef.h>
#include <string.h>
/* A stand-in for libnccl: ncclGetUniqueId fails when FAIL_ID is defined, ncclCommInitRank always fails. */
typedef struct { char internal[128]; } ncclUniqueId;
int ncclGetUniqueId(ncclUniqueId* id) {
#ifdef FAIL_ID
    (void)id; return 3;
#else
    memset(id, 7, sizeof(*id)); return 0;
#endif
}
int ncclCommInitRank(void** comm, int nranks, ncclUniqueId id, int rank) { (void)comm; (void)nranks; (void)id; (void)rank; return 5; }
int ncclBroadcast(const void* s, void* r, size_t n, int dt, int root, void* comm, void* stream) { return 5; }
#ifndef NO_ALLGATHER
int ncclAllGather(const void* s, void* r, size_t n, int dt, void* comm, void* stream) { return 5; }
#endif
int ncclCommDestroy(void* comm) { (void)comm; return 0; }
const char* ncclGetErrorString(int rc) { (void)rc; return "stand-in NCCL: injected failure"; }
"""

CHILD = r"""
import ctypes as C, sys
L = C.CDLL(sys.argv[1])
L.b200wmma_last_error_string.restype = C.c_char_p
buf = C.create_string_buffer(128)
rc_id = L.b200wmma_mg_unique_id(buf)
msg_id = L.b200wmma_last_error_string().decode()
h = C.c_void_p(1234)
rc_cr = L.b200wmma_mg_create(C.byref(h), buf, 0, 2)
msg_cr = L.b200wmma_last_error_string().decode()
print("ID", rc_id, msg_id)
print("CREATE", rc_cr, h.value, msg_cr)
"""


def _build_fake(tmp_path, name, defs=()):
    src = tmp_path / (name + ".c")
    src.write_text(FAKE_NCCL)
    out = tmp_path / (name + ".so")
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", *defs, str(src), "-o", str(out)], check=True)
    return str(out)


def _child(tmp_path, nccl_path):
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    env = dict(os.environ, B200WMMA_NCCL_LIBRARY=nccl_path)
    res = subprocess.run([sys.executable, str(script), _lib.LIB_PATH], capture_output=True, text=True, env=env, timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr
    lines = dict(l.split(" ", 1) for l in res.stdout.strip().splitlines())
    return lines["ID"], lines["CREATE"]


@pytest.fixture(autouse=True)
def _needs_library():
    if not os.path.exists(_lib.LIB_PATH):
        pytest.skip("librocwmma_b200.so not built")


def test_nccl_library_that_cannot_be_opened(tmp_path):
    missing = str(tmp_path / "no_such_nccl.so")
    id_line, create_line = _child(tmp_path, missing)
    assert id_line.startswith("2 ") and "B200WMMA_NCCL_LIBRARY" in id_line and "no_such_nccl.so" in id_line
    rc, handle, _ = create_line.split(" ", 2)
    assert rc == "2" and handle == "None"      # UNSUPPORTED, and the out handle was cleared


def test_nccl_library_without_a_needed_symbol(tmp_path):
    fake = _build_fake(tmp_path, "fake_nccl_nosym", ["-DNO_ALLGATHER"])
    id_line, create_line = _child(tmp_path, fake)
    assert id_line.startswith("2 ") and "ncclAllGather" in id_line
    assert create_line.startswith("2 None")


def test_nccl_unique_id_call_that_fails(tmp_path):
    fake = _build_fake(tmp_path, "fake_nccl_failid", ["-DFAIL_ID"])
    id_line, _ = _child(tmp_path, fake)
    assert id_line.startswith("2 ") and "injected failure" in id_line


@pytest.mark.gpu
def test_nccl_comm_init_that_fails(tmp_path):
    """ncclCommInitRank returns an error (stand-in library): no handle, B200WMMA_ERR_UNSUPPORTED, the cause in the
    message; the rest of the library is unaffected.  Needs a device only because mg_create asks which one is current."""
    fake = _build_fake(tmp_path, "fake_nccl_failinit")
    id_line, create_line = _child(tmp_path, fake)
    assert id_line.startswith("0 ")
    rc, handle, msg = create_line.split(" ", 2)
    assert rc == "2" and handle == "None" and "ncclCommInitRank failed" in msg and "injected failure" in msg
