"""The reference's own symbol, cuda_flash_attention_fwd, served by liblogos_attn_shim.so: a C++
program that knows only the reference's declaration is compiled, linked against the shim and run."""
import os
import subprocess

import numpy as np
import pytest

import oracle as O
from logos_b200 import synthetic as syn
from logos_b200.build import PKG
from helpers import assert_close

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def driver(tmp_path_factory):
    exe = str(tmp_path_factory.mktemp("shim") / "shim_driver")
    subprocess.check_call(["nvcc", "-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-o", exe,
                           os.path.join(HERE, "shim_driver.cu"), "-L" + PKG, "-llogos_attn_shim", "-llogos_attn",
                           "-Xlinker", "-rpath=" + PKG])
    return exe


@pytest.mark.parametrize("seq,window,stride", [(200, 0, 0), (333, 64, 16)])
def test_drop_in_symbol_matches_the_cpu_model(driver, tmp_path, seq, window, stride):
    DH = 64
    q, k, v = (syn.normal((seq, DH), 71, t) for t in (1, 2, 3))
    np.concatenate([q, k, v]).astype(np.float32).tofile(str(tmp_path / "in.bin"))
    res = subprocess.run([driver, str(tmp_path / "in.bin"), str(tmp_path / "out.bin"), str(seq), str(DH),
                          str(window), str(stride)], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stderr
    assert res.stdout.startswith("rejected: "), res.stdout          # DH = 256 must throw, as in the reference
    got = np.fromfile(str(tmp_path / "out.bin"), dtype=np.float32).reshape(seq, DH)
    p = O.attn_params(0.125, True, window, stride, 0.0, 0.0, 0.0, O.DIFFUSE_NONE)
    want = O.attention_rows(q, k, v, p)
    assert_close(got, want, f"shim seq={seq} window={window}", 2e-5, 1e-5)
