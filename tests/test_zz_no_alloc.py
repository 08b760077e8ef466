"""The decode entry point for callers that cannot allocate (logos_decode_int8_noalloc).

Such callers -- a host whose memory pool owns the whole device, a serving loop that
forbids allocation after start-up, an embedding without a logos_ctx -- get the split-K
scratch from a fixed array inside the library.  The test drives the entry point through
the C ABI, twice in a row on different inputs (the array keeps the first call's
contents), and compares with the context-based entry point and with the CPU oracle.  It lives in
a file that is collected last, and it passes on its own in a fresh process as well as after the others.

Where the library's device code gets its memory: CUDA loads a library's kernels and __device__ arrays
into a device on first use.  For a process that never made a logos_ctx, the first call of this entry
point IS that first use, so it -- and only it -- takes device memory (the kernel image and the 4.3 MB
array).  A caller whose pool is about to take the whole device makes one warm-up call before that;
the last test below checks, in a process of its own, that the second call moves nothing.
"""
import ctypes as C
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest
import torch

import oracle as O
from logos_b200 import lib as L
from helpers import assert_close

pytestmark = pytest.mark.gpu


def _inputs(B, H, S, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    kq = torch.randint(-127, 128, (B, H, S, 64), dtype=torch.int8, device="cuda", generator=g)
    vq = torch.randint(-127, 128, (B, H, S, 64), dtype=torch.int8, device="cuda", generator=g)
    ks = torch.rand((B, H), device="cuda", generator=g) * 0.02 + 0.01
    vs = torch.rand((B, H), device="cuda", generator=g) * 0.02 + 0.01
    q = torch.randn((B, H, 64), device="cuda", generator=g).half()
    qp = torch.randn((B, H, 64), device="cuda", generator=g).half()
    lens = torch.randint(1, S + 1, (B,), dtype=torch.int32, device="cuda", generator=g)
    lens[0] = S
    return q, qp, kq, vq, ks, vs, lens


def _noalloc(lib, q, qp, kq, vq, ks, vs, lens, p, out=None):
    B, H, S, DH = kq.shape
    if out is None:
        out = torch.full((B, H, DH), float("nan"), device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.logos_decode_int8_noalloc(C.c_void_p(stream), q.data_ptr(), qp.data_ptr(), kq.data_ptr(), vq.data_ptr(),
                                       ks.data_ptr(), vs.data_ptr(), lens.data_ptr(), B, H, S, DH, C.byref(p),
                                       out.data_ptr())
    return rc, out


def _oracle(q, qp, kq, vq, ks, vs, lens, p):
    B, H, S, DH = kq.shape
    n = B * H
    op = O.attn_params(p.scale, p.causal, p.window, p.stride, p.ns_eta, p.ns_nu, p.ns_alpha, p.diffuse_mode)
    return O.decode_int8_batch(q.float().cpu().numpy().reshape(n, DH), qp.float().cpu().numpy().reshape(n, DH),
                               kq.cpu().numpy().reshape(n, S, DH), vq.cpu().numpy().reshape(n, S, DH),
                               ks.cpu().numpy().reshape(n), vs.cpu().numpy().reshape(n),
                               np.repeat(lens.cpu().numpy(), H), op).reshape(B, H, DH)


def test_noalloc_matches_context_entry_point_twice(engine):
    lib = L.load_library()
    cases = [(L.Params.make(0.125, True, 0, 0, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL), 8, 4, 4096, 1),
             (L.Params.make(0.125, True, 0, 0, 0.1, 0.05, 0.3, L.DIFFUSE_CENTRAL), 3, 5, 2048, 2)]
    for p, B, H, S, seed in cases:          # two calls in a row, different shapes and inputs
        args = _inputs(B, H, S, seed)
        engine.reserve(engine.decode_workspace_bytes(B, H, S, 64))
        want = engine.decode_int8(*args, p)
        got = torch.full((B, H, 64), float("nan"), device="cuda")
        free_before = torch.cuda.mem_get_info()[0]
        rc, got = _noalloc(lib, *args, p, out=got)
        torch.cuda.synchronize()
        assert rc == L.OK, lib.logos_status_string(rc)
        assert torch.cuda.mem_get_info()[0] == free_before     # the device's free memory did not move
        assert_close(got.cpu().numpy(), want.cpu().numpy(), f"noalloc case {seed}", 1e-5, 1e-5)
        assert_close(got.cpu().numpy(), _oracle(*args, p), f"noalloc case {seed} vs oracle")
    # same inputs again: the scratch still holds the previous call's records
    rc, again = _noalloc(lib, *args, p)
    assert rc == L.OK and torch.equal(again, got)


def test_noalloc_limits_are_reported(engine):
    lib = L.load_library()
    p = L.Params.make(0.125, True, 0, 0, 0.0, 0.0, 1.0, L.DIFFUSE_NONE)
    one = torch.zeros(1, device="cuda")
    d = one.data_ptr()
    # 8192 pairs exceed the 4096-pair limit; nothing is launched, so tiny buffers are fine
    assert lib.logos_decode_int8_noalloc(None, d, d, d, d, d, d, d, 512, 16, 64, 64, C.byref(p), d) == L.ERR_SCRATCH_LIMIT
    # 4096 pairs x 8 splits exceed the 16384-record limit
    assert lib.logos_decode_int8_noalloc(None, d, d, d, d, d, d, d, 256, 16, 8192, 64, C.byref(p), d) == L.ERR_SCRATCH_LIMIT
    pw = L.Params.make(0.125, True, 64, 16, 0.0, 0.0, 1.0, L.DIFFUSE_NONE)
    assert lib.logos_decode_int8_noalloc(None, d, d, d, d, d, d, d, 1, 1, 64, 64, C.byref(pw), d) == L.ERR_UNSUPPORTED
    assert b"scratch" in lib.logos_status_string(L.ERR_SCRATCH_LIMIT)


def test_noalloc_in_a_process_without_a_context():
    """A fresh process that never creates a logos_ctx: the first call loads the library's device code
    (that is where its memory comes from), the second call moves no device memory, and both match the
    CPU oracle."""
    root = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
    code = textwrap.dedent("""
        import ctypes as C, sys
        sys.path.insert(0, %r); sys.path.insert(0, %r)
        import numpy as np, torch
        import oracle as O
        from logos_b200 import lib as L
        from test_zz_no_alloc import _inputs, _noalloc, _oracle
        lib = L.load_library()
        p = L.Params.make(0.125, True, 0, 0, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL)
        args = _inputs(4, 4, 4096, 3)
        want = _oracle(*args, p)
        torch.cuda.synchronize()
        rc, first = _noalloc(lib, *args, p)          # warm-up: module load happens here
        torch.cuda.synchronize()
        assert rc == L.OK, rc
        out = torch.full((4, 4, 64), float("nan"), device="cuda")
        free_before = torch.cuda.mem_get_info()[0]
        rc, second = _noalloc(lib, *args, p, out=out)
        torch.cuda.synchronize()
        assert rc == L.OK, rc
        assert torch.cuda.mem_get_info()[0] == free_before, "the second call moved device memory"
        for got in (first, second):
            err = float(np.abs(got.cpu().numpy() - want).max())
            assert err < 2e-3, err
        print("ok")
    """ % (root, os.path.join(root, "tests")))
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and res.stdout.strip().endswith("ok"), res.stdout + res.stderr
