"""tcq_encode_tb_static: the encoder for callers that cannot allocate device memory.

A host that has handed its whole device budget to another framework cannot produce the workspace tcq_encode_tb wants.  The static entry point keeps
its scratch in a fixed array of the library image instead.  It must give exactly what the
ordinary entry point gives, call after call (the array is reused and never cleared), and must
refuse batches that do not fit.

Collected last on purpose (file name), so a run that stops at the first failure has already
gone through every other test.
"""
import numpy as np
import pytest
import torch

from conftest import same_bits

pytestmark = pytest.mark.gpu


def _encode(lib, fn_static, w, K, cid):
    n = w.shape[0]
    packed = torch.zeros(n, 8 * K, dtype=torch.int32, device="cuda")
    bits = torch.zeros(n, 256, dtype=torch.int64, device="cuda")
    dq = torch.zeros(n, 256, device="cuda")
    sse = torch.zeros(n, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    if fn_static:
        rc = lib.tcq_encode_tb_static(w.data_ptr(), n, K, cid, packed.data_ptr(), bits.data_ptr(), dq.data_ptr(),
                                      sse.data_ptr(), stream)
    else:
        ws = torch.empty(int(lib.tcq_workspace_bytes(n, K)), dtype=torch.uint8, device="cuda")
        rc = lib.tcq_encode_tb(w.data_ptr(), n, K, cid, packed.data_ptr(), bits.data_ptr(), dq.data_ptr(),
                               sse.data_ptr(), ws.data_ptr(), ws.numel(), stream)
    torch.cuda.synchronize()
    return rc, packed, bits, dq, sse


@pytest.mark.parametrize("K,cid", [(3, 1), (2, 2), (4, 0)])
def test_static_scratch_encoder_matches_workspace_encoder_twice(K, cid, oracle, luts):
    from trellis_b200 import _lib
    lib = _lib.lib()
    assert torch.cuda.is_available()
    n = int(lib.tcq_encode_tb_static_max_tiles(K))
    assert {2: 31, 3: 42, 4: 63}[K] == n
    g = torch.Generator(device="cuda").manual_seed(100 + K)
    name = ("1mad", "3inst", "mcg")[cid]
    for call in range(2):                                   # second call runs on the first call's leftovers
        w = torch.randn(n - 5 * call, 256, generator=g, device="cuda") * 1.2
        rc_s, *out_s = _encode(lib, True, w, K, cid)
        rc_w, *out_w = _encode(lib, False, w, K, cid)
        assert rc_s == 0 and rc_w == 0
        for a, b in zip(out_s, out_w):                      # packed words, symbols, reconstruction, squared error
            assert torch.equal(a, b)                        # bit-exact: same kernels, only the scratch differs
        # and against the CPU oracle directly, so that this file does not lean on the other entry point alone
        bits, dq, sse = oracle.viterbi_tb(w[:6].cpu().numpy(), K, luts[name], with_sse=True)
        assert np.array_equal(out_s[1][:6].cpu().numpy(), bits)
        assert same_bits(out_s[2][:6].cpu().numpy(), dq) and same_bits(out_s[3][:6].cpu().numpy(), sse)
        assert lib.tcq_encode_tb_static_status(torch.cuda.current_stream().cuda_stream) == 0


def test_static_scratch_encoder_allocates_nothing_and_reports_its_status():
    """Device memory in use does not move across a call (after the first, which resolves the array's address), and the
    status word inside the array is readable through tcq_encode_tb_static_status."""
    from trellis_b200 import _lib
    lib = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    w = torch.randn(12, 256, device="cuda")
    packed = torch.empty(12, 24, dtype=torch.int32, device="cuda")
    assert lib.tcq_encode_tb_static(w.data_ptr(), 12, 3, 2, packed.data_ptr(), None, None, None, stream) == 0
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert lib.tcq_encode_tb_static(w.data_ptr(), 12, 3, 2, packed.data_ptr(), None, None, None, stream) == 0
    assert lib.tcq_encode_tb_static_status(stream) == 0             # synchronises
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    bad = w.clone()
    bad[3, 5] = float("inf")
    assert lib.tcq_encode_tb_static(bad.data_ptr(), 12, 3, 2, packed.data_ptr(), None, None, None, stream) == 0
    assert lib.tcq_encode_tb_static_status(stream) == -11           # TCQ_E_NONFINITE_INPUT: flagged, never trapped on
    assert lib.tcq_encode_tb_static(w.data_ptr(), 12, 3, 2, packed.data_ptr(), None, None, None, stream) == 0
    assert lib.tcq_encode_tb_static_status(stream) == 0             # the flag is per call


def test_static_scratch_encoder_refuses_oversized_batches():
    from trellis_b200 import _lib
    lib = _lib.lib()
    n = int(lib.tcq_encode_tb_static_max_tiles(3)) + 1
    w = torch.randn(n, 256, device="cuda")
    packed = torch.full((n, 24), 7, dtype=torch.int32, device="cuda")
    rc = lib.tcq_encode_tb_static(w.data_ptr(), n, 3, 1, packed.data_ptr(), None, None, None,
                                  torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == -9 and b"static scratch" in lib.tcq_strerror(rc)
    assert int((packed != 7).sum()) == 0                    # nothing was launched
    assert lib.tcq_encode_tb_static(w.data_ptr(), 1, 7, 1, packed.data_ptr(), None, None, None, None) == -1
    assert lib.tcq_encode_tb_static(w.data_ptr(), 0, 3, 1, packed.data_ptr(), None, None, None, None) == 0
