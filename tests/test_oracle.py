"""The CPU oracle (oracle/tcq_oracle.c) against the reference's own outputs and known answers.

These pin the oracle: every array in tests/golden/ was produced by running the reference's
Python code (tests/golden/make_golden.py), and the oracle must reproduce it bit for bit.
"""
import hashlib

import numpy as np
import pytest

from conftest import CODEBOOKS, KS, same_bits


def test_1mad_known_answer(oracle):
    # tests/test_qtip.py:23-27 of the reference: state 0 -> LCG word 0x0491367A, byte sum 325
    v = oracle.codebook_lut("1mad")[0]
    assert abs(float(v) - (325 - 510) / 147.800537109375) < 1e-6


@pytest.mark.parametrize("name", CODEBOOKS)
def test_codebook_tables_match_reference(oracle, golden, name):
    lut = oracle.codebook_lut(name)
    assert lut.shape == (65536,) and lut.dtype == np.float32
    sha = np.frombuffer(hashlib.sha256(lut.tobytes()).digest(), dtype=np.uint8)
    assert np.array_equal(sha, golden["codebooks"][f"{name}_sha256"])
    assert same_bits(lut[::251], golden["codebooks"][f"{name}_sample"])
    # tests/test_qtip.py:29-32: roughly standard normal over all states
    assert abs(float(lut.mean())) < 0.05 and 0.8 < float(lut.std()) < 1.35


@pytest.mark.parametrize("K", KS)
@pytest.mark.parametrize("name", CODEBOOKS)
def test_viterbi_passes_match_reference(oracle, golden, luts, name, K):
    g = golden["encode"]
    w = g["w"]
    key = f"{name}_K{K}"
    s1 = oracle.viterbi_pass(np.roll(w, 128, axis=1), K, luts[name], None)
    assert np.array_equal(s1, g[key + "_states1"].astype(np.int64))
    ov = (s1[:, 128] >> K).astype(np.int32)
    assert np.array_equal(ov, g[key + "_overlap"])
    s2 = oracle.viterbi_pass(w, K, luts[name], ov)
    assert np.array_equal(s2, g[key + "_states2"].astype(np.int64))


@pytest.mark.parametrize("K", KS)
@pytest.mark.parametrize("name", CODEBOOKS)
def test_viterbi_tb_matches_reference(oracle, golden, luts, name, K):
    g = golden["encode"]
    bits, dq, sse = oracle.viterbi_tb(g["w"], K, luts[name], with_sse=True)
    key = f"{name}_K{K}"
    assert np.array_equal(bits, g[key + "_bits"].astype(np.int64))
    assert same_bits(dq, g[key + "_dq"])
    assert np.allclose(sse, ((g["w"] - dq) ** 2).sum(axis=1), rtol=1e-5)
    assert int(bits.max()) < (1 << K)


def test_viterbi_tb_on_incoherence_processed_tiles(oracle, golden, luts):
    g = golden["encode_ip"]
    bits, dq = oracle.viterbi_tb(g["w"], 3, luts["3inst"])
    assert np.array_equal(bits, g["bits"].astype(np.int64))
    assert same_bits(dq, g["dq"])


def test_thread_count_does_not_change_results(oracle, golden, luts):
    w = golden["encode"]["w"]
    a = oracle.viterbi_tb(w, 3, luts["mcg"], nthreads=1)
    b = oracle.viterbi_tb(w, 3, luts["mcg"], nthreads=4)
    assert np.array_equal(a[0], b[0]) and same_bits(a[1], b[1])


@pytest.mark.parametrize("K", KS)
@pytest.mark.parametrize("name", CODEBOOKS)
def test_decode_matches_reference(oracle, golden, luts, name, K):
    g = golden["decode"]
    bits = g[f"K{K}_bits"].astype(np.int64)
    s0 = g[f"K{K}_s0"]
    lut = luts[name]
    assert same_bits(oracle.decode_recursive(bits, K, lut), g[f"{name}_K{K}_recursive"])
    assert same_bits(oracle.decode_window(bits, K, lut), g[f"{name}_K{K}_window"])
    assert same_bits(oracle.decode_recursive(bits, K, lut, s0), g[f"{name}_K{K}_recursive_s0"])
    assert same_bits(oracle.decode_window(bits, K, lut, s0), g[f"{name}_K{K}_window_s0"])


@pytest.mark.parametrize("K", KS)
def test_packing_and_wrapped_decode(oracle, golden, luts, K):
    enc = golden["encode"]
    bits = enc[f"mcg_K{K}_bits"].astype(np.int64)
    packed = oracle.pack_bits(bits, K)
    assert packed.shape == (bits.shape[0], 8 * K)
    assert np.array_equal(packed, golden["decode"][f"K{K}_packed"])          # the reference's pack_bits_np
    # tests/test_qtip.py:55-67: the wrapped stream alone reproduces the encoder's reconstruction ...
    assert same_bits(oracle.decode_wrapped(bits, K, luts["mcg"]), enc[f"mcg_K{K}_dq"])
    # ... and so does the window decode of the packed words (web/kernels.js wz())
    assert same_bits(oracle.decode_packed(packed, K, "mcg"), enc[f"mcg_K{K}_dq"])


def test_k2_distortion_on_gaussian(oracle, luts):
    # tests/test_qtip.py:71-83: K=2 trellis MSE on N(0,1) stays below 0.085
    rng = np.random.default_rng(2)
    w = rng.standard_normal((16, 256)).astype(np.float32)
    _, dq = oracle.viterbi_tb(w, 2, luts["mcg"])
    assert float(((w - dq) ** 2).mean()) < 0.085


def test_encoding_a_reconstruction_is_lossless(oracle, golden, luts):
    dq = golden["encode"]["3inst_K3_dq"]
    _, dq2, sse = oracle.viterbi_tb(dq, 3, luts["3inst"], with_sse=True)
    assert same_bits(dq, dq2) and float(sse.max()) == 0.0


# First 16 hex digits of sha256(symbols as uint8, row-major) that the reference's ``viterbi_tb(w, K, lut)`` (fp32 DP,
# torch CPU) gives on ``torch.manual_seed(0); w = torch.randn(256, 256)[:64]``, written down from a run of the
# reference that was independent of the one that made tests/golden/encode.npz.
REFERENCE_SYMBOL_DIGESTS = {
    ("1mad", 2): "eeb3b7fceca53b36", ("1mad", 3): "c53c13668c3c4bd2", ("1mad", 4): "a208c9b2c9f09a1b",
    ("3inst", 2): "f06b0c366c4357ba", ("3inst", 3): "116385363d10203d", ("3inst", 4): "160b4edf586c89af",
    ("mcg", 2): "e2986c2f4e9e1b5d", ("mcg", 3): "385e33af294e2021", ("mcg", 4): "0d559459225b0b63",
}


@pytest.mark.parametrize("K", KS)
@pytest.mark.parametrize("name", CODEBOOKS)
def test_viterbi_tb_matches_reference_on_64_tiles(oracle, golden, luts, name, K):
    g = golden["encode"]
    w = g["w64"]
    assert w.shape == (64, 256) and np.array_equal(w[:6], g["w"])
    bits, dq = oracle.viterbi_tb(w, K, luts[name])
    key = f"{name}_K{K}"
    assert np.array_equal(bits, g[key + "_bits64"].astype(np.int64))
    sha = np.frombuffer(hashlib.sha256(np.ascontiguousarray(dq).tobytes()).digest(), dtype=np.uint8)
    assert np.array_equal(sha, g[key + "_dq64_sha256"])
    assert hashlib.sha256(bits.astype(np.uint8).tobytes()).hexdigest()[:16] == REFERENCE_SYMBOL_DIGESTS[(name, K)]


def test_viterbi_tb_on_tiles_of_the_second_configuration(oracle, golden, luts):
    """16 tiles spread over the 4096 x 4096 outlier matrix, exactly as the reference's IPContext made them."""
    g = golden["cfg2_probe"]
    assert g["tiles"].shape == (16, 256) and int(g["index"][-1]) == 65535
    bits, dq = oracle.viterbi_tb(g["tiles"], 3, luts["3inst"])
    assert np.array_equal(bits, g["bits"].astype(np.int64))
    assert same_bits(dq, g["dq"])
