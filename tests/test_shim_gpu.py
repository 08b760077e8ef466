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


def test_reference_model_forward_with_the_drop_in_symbol(tmp_path):
    """The reference's ModelGPU::forward (cuda/ModelGPU.cu, compiled unchanged) on a small seeded model,
    once with the reference's own cuda_flash_attention_fwd and once linked against liblogos_attn_shim.so
    (the reference's definition renamed away at compile time of cuda/VedicGEMM.cu): the logits agree.
    Shunyam is active (seq > window), so the drop-in also has to honour window and stride."""
    stock, dropin = O.refmodel("stock"), O.refmodel("dropin")
    if stock is None or dropin is None:
        pytest.skip("oracle/_ref/refmodel_* were not built (reference tree absent at build time)")
    args = ["96", "128", "2", "2", "150", "32", "8"]          # vocab d_model heads layers seq window stride
    env = dict(os.environ, LD_LIBRARY_PATH=PKG + ":" + os.environ.get("LD_LIBRARY_PATH", ""))
    outs = []
    for exe, name in ((stock, "stock.bin"), (dropin, "dropin.bin")):
        res = subprocess.run([exe, str(tmp_path / name), *args], capture_output=True, text=True, timeout=300, env=env)
        assert res.returncode == 0, res.stderr[-2000:]
        outs.append(np.fromfile(str(tmp_path / name), dtype=np.float32).reshape(150, 96))
    assert np.isfinite(outs[0]).all() and np.abs(outs[0]).max() > 1e-3
    assert_close(outs[1], outs[0], "logits with the drop-in symbol vs the reference's own kernel", 2e-4, 1e-4)
