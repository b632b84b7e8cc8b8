"""Per-instruction parity on the GPU: every opcode, through the C ABI, against the C
oracle on the same seeded bytes. Tolerance for FP32-accumulated math is the stated
rel 1e-3 / abs 1e-4 (most cases are pinned much tighter, or bit-exact where the
arithmetic is order-free); integer / gather work is bit-exact. Canary bytes around
every operand must survive: no kernel may write outside its outputs."""
import numpy as np
import pytest

import opcases
from oracle import pyoracle as O

pytestmark = pytest.mark.gpu


def _run_case(c, gemm):
    from see_ml_b200.engine import Context
    want = c.arena.copy()
    O.execute("port", c.instr, want, c.rodata, **c.scalars)
    ctx = Context(c.arena.size, c.rodata, gemm=gemm)
    ctx.write(0, c.arena)
    ctx.execute(c.instr, **c.scalars)
    got = ctx.read(0, c.arena.size)
    ctx.close()
    return want, got


def _compare(c, want, got):
    mask = np.ones(c.arena.size, bool)
    for name, spec in c.outputs.items():
        off, count, dt = spec
        mask[off:off + 4 * count] = False
        w, g = opcases.read_output(want, spec), opcases.read_output(got, spec)
        if c.exact:
            np.testing.assert_array_equal(g.view(np.uint32), w.view(np.uint32), err_msg=f"{c.name}/{name}")
        else:
            nan_w, nan_g = np.isnan(w), np.isnan(g)
            np.testing.assert_array_equal(nan_g, nan_w, err_msg=f"{c.name}/{name}: NaN pattern")
            np.testing.assert_allclose(g[~nan_w], w[~nan_w], rtol=c.rtol, atol=c.atol,
                                       err_msg=f"{c.name}/{name}")
    np.testing.assert_array_equal(got[mask], want[mask], err_msg=f"{c.name}: bytes outside the outputs changed")


@pytest.mark.parametrize("family", ["elementwise", "norm", "attention", "loss", "optimizer"])
def test_family_matches_oracle(family):
    rng = np.random.default_rng(4321)
    cases = getattr(opcases, family + "_cases")(rng)
    assert len(cases) > 5
    for c in cases:
        want, got = _run_case(c, gemm=0)
        _compare(c, want, got)


@pytest.mark.parametrize("gemm", [0, 2], ids=["tf32x3", "fp32_simt"])
def test_gemm_family_matches_oracle(gemm):
    rng = np.random.default_rng(99)
    for c in opcases.gemm_cases(rng, big=True):
        want, got = _run_case(c, gemm=gemm)
        _compare(c, want, got)


@pytest.mark.parametrize("gemm", [0, 2], ids=["tf32x3", "fp32_simt"])
def test_attention_family_large_shapes(gemm):
    """Sequence lengths that are multiples of 128 with 64-wide heads take the batched
    tensor-core kernel (3xTF32, transposed operands re-laid in shared memory); the CUDA-core
    kernel is held to the tight per-case tolerance, the tensor-core one to the stated one."""
    rng = np.random.default_rng(5)
    for c in opcases.attention_cases(rng, big=True)[-14:]:
        want, got = _run_case(c, gemm=gemm)
        if gemm == 0 and c.name.startswith("ATTN_"):
            c.rtol, c.atol = max(c.rtol, 1e-3), max(c.atol, 1e-4)
        _compare(c, want, got)


def test_masked_entries_stay_exact_zeros_on_the_tensor_core_path():
    rng = np.random.default_rng(9)
    cases = opcases.attention_cases(rng, big=True)
    for prefix, key in (("ATTN_FWD_1x512", "P"), ("ATTN_DP_1x512", "dP")):
        c = next(c for c in cases if c.name.startswith(prefix))
        _, got = _run_case(c, gemm=0)
        P = opcases.read_output(got, c.outputs[key]).reshape(-1, 512, 512)
        iu = np.triu_indices(512, 1)
        assert np.all(P[:, iu[0], iu[1]] == 0.0), prefix


def test_masked_attention_entries_are_exact_zeros():
    rng = np.random.default_rng(8)
    c = next(c for c in opcases.attention_cases(rng) if c.name.startswith("ATTN_FWD_2x64"))
    _, got = _run_case(c, gemm=0)
    P = opcases.read_output(got, c.outputs["P"]).reshape(-1, 64, 64)
    assert np.all(P[:, np.triu_indices(64, 1)[0], np.triu_indices(64, 1)[1]] == 0.0)
    np.testing.assert_allclose(P.sum(-1), 1.0, rtol=1e-5)


def test_kernels_are_run_to_run_bit_reproducible():
    rng = np.random.default_rng(3)
    for c in opcases.gemm_cases(rng, big=True)[-6:] + opcases.loss_cases(rng)[:8] + opcases.norm_cases(rng)[:8]:
        _, a = _run_case(c, gemm=0)
        _, b = _run_case(c, gemm=0)
        np.testing.assert_array_equal(a, b, err_msg=c.name)
