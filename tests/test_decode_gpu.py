"""Device-resident decode step against the CPU restatement (tests/decode_ref.py)."""
import copy

import numpy as np
import pytest

from demonic_b200 import _lib, decoder
from tests import decode_ref
from tests.parity import assert_parity

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[1, 0], ids=["fused", "one_kernel_per_op"], autouse=True)
def arrangement(request):
    """Both launch sequences of the same step: companions fused into the GEMVs / attention, or one kernel per op."""
    lib = _lib.load()
    lib.dmc_cuda_clear_error()
    lib.dmc_cuda_set_param(b"decode_fused", request.param)
    yield
    lib.dmc_cuda_set_param(b"decode_fused", 1)


def run_case(cfg, cache_len, tokens):
    model = decoder.random_model(cfg, seed=99, cache_len=cache_len)
    ref_model = copy.deepcopy(model)
    dec = decoder.Decoder(cfg, model)
    try:
        pos = cache_len
        for tok in tokens:
            nxt, logits = dec.step(tok, pos, want_logits=True)
            rnxt, rlogits = decode_ref.step(cfg, ref_model, tok, pos)
            # companions are tolerance-matched (rtol 1e-3 / atol 1e-4 class, tools/numpy_oracle.py:41-42)
            assert_parity(logits, rlogits, 1e-2, f"logits at pos {pos}")
            assert nxt == rnxt or abs(rlogits[nxt] - rlogits[rnxt]) < 1e-4 * max(1.0, abs(rlogits[rnxt])), "token differs"
            assert nxt == int(np.argmax(logits))
            pos += 1
    finally:
        dec.close()
    assert _lib.load().dmc_cuda_status() == 0


def test_small_model_several_steps():
    cfg = decoder.Config(layers=2, d_model=256, heads=2, head_dim=128, ffn=520, vocab=1003, max_len=40)
    run_case(cfg, cache_len=17, tokens=[5, 1002, 0, 77])


def test_empty_cache_first_token():
    cfg = decoder.Config(layers=1, d_model=128, heads=1, head_dim=128, ffn=128, vocab=64, max_len=8)
    run_case(cfg, cache_len=0, tokens=[3, 9])


def test_benchmark_configuration_one_step():
    cfg = decoder.Config()                      # 8 layers, d_model 2048, 16x128 heads, FFN 5632, vocab 32000
    run_case(cfg, cache_len=512, tokens=[1234])


def test_token_ids_clamp_like_embed():
    cfg = decoder.Config(layers=1, d_model=128, heads=1, head_dim=128, ffn=128, vocab=64, max_len=8)
    model = decoder.random_model(cfg, seed=5, cache_len=2)
    dec = decoder.Decoder(cfg, model)
    a = dec.step(10 ** 6, 2, want_logits=True)[1]
    b = dec.step(cfg.vocab - 1, 2, want_logits=True)[1]
    assert np.array_equal(a, b)
    dec.close()
