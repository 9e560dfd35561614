"""CPU-side checks: the C-ABI library loads and exports what the header declares, argument
validation, the host logic of LDLQ / incoherence processing, and the multi-rank plumbing (gloo)."""
import ctypes
import os
import re
import zlib

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT

from trellis_b200 import _lib, dist as tdist, ldlq, qtip


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "tcq_b200.h")).read()
    return re.findall(r"TCQ_API[^;(]*?\b(tcq_\w+)\s*\(", text)


def test_library_exports_every_declared_symbol():
    names = _declared_symbols()
    assert len(names) >= 11
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), f"{n} is declared in include/tcq_b200.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes signatures and header are out of step"
    assert _lib.lib().tcq_abi_version() == _lib.ABI_VERSION


def test_error_strings_and_workspace_sizes():
    L = _lib.lib()
    for code in range(0, -9, -1):
        assert L.tcq_strerror(code)
    assert L.tcq_workspace_min_bytes(5) == 0 and L.tcq_workspace_bytes(10, 1) == 0
    for K, per_tile in ((2, 1 << 20), (3, 768 << 10), (4, 512 << 10)):     # 256 steps x E*K/8 bytes
        assert per_tile <= L.tcq_workspace_min_bytes(K) < per_tile + 4096
        assert L.tcq_workspace_bytes(100, K) >= 100 * per_tile
        assert L.tcq_workspace_bytes(10 ** 7, K) < 8 << 30                # chunked, not proportional to n


def test_argument_validation_needs_no_gpu():
    L = _lib.lib()
    buf = (ctypes.c_char * 4096)()
    p = ctypes.addressof(buf)
    p += (-p) % 256
    assert L.tcq_encode_tb(p, 1, 5, 0, p, None, None, None, p, 4096, None) == -1       # K
    assert L.tcq_encode_tb(p, 1, 3, 7, p, None, None, None, p, 4096, None) == -2       # codebook
    assert L.tcq_encode_tb(p, -1, 3, 0, p, None, None, None, p, 4096, None) == -3      # count
    assert L.tcq_encode_tb(None, 1, 3, 0, p, None, None, None, p, 4096, None) == -4    # NULL input
    assert L.tcq_encode_tb(p + 4, 1, 3, 0, p, None, None, None, p, 4096, None) == -5   # misaligned input
    assert L.tcq_encode_tb(p, 0, 3, 0, None, None, None, None, None, 0, None) == 0     # empty batch is a no-op
    assert L.tcq_viterbi_pass(p, 1, 3, 0, None, 7, p, p, 4096, None) == -8             # roll
    assert L.tcq_decode_packed(None, 1, 3, 0, p, None) == -4
    assert L.tcq_decode_symbols(p, 1, -1, 3, 0, None, p, None) == -3
    assert L.tcq_pack_symbols(p, 1, 9, p, None) == -1
    assert L.tcq_codebook_lut(3, p, None) == -2


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the behaviour on a box without a GPU")
def test_product_path_fails_loudly_without_gpu():
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        qtip.encode(torch.zeros(1, 256), 3, "mcg")
    with pytest.raises(RuntimeError):
        qtip.codebook_lut("mcg")


def test_encode_rejects_bad_shapes_before_touching_the_device():
    with pytest.raises(ValueError):
        qtip.encode(torch.zeros(2, 128), 3, "mcg")
    with pytest.raises(ValueError):
        qtip.encode(torch.zeros(2, 256), 5, "mcg")
    with pytest.raises(ValueError):
        qtip.pack_bits(torch.zeros(2, 100, dtype=torch.long), 3)


def test_tiling_matches_reference_index_map():
    # qtip.py:288 / :303: tile = (row/16)*(k/16) + col/16, t = (row%16)*16 + col%16
    n, k = 32, 48
    z = torch.arange(n * k, dtype=torch.float32).reshape(n, k)
    tiles = qtip.to_tiles(z)
    assert tiles.shape == (n // 16 * k // 16, 256)
    for row, col in ((0, 0), (5, 17), (31, 47), (16, 15)):
        assert tiles[(row // 16) * (k // 16) + col // 16, (row % 16) * 16 + col % 16] == z[row, col]
    assert torch.equal(qtip.from_tiles(tiles, n, k), z)


def test_incoherence_processing_round_trip():
    # tests/test_qtip.py:86-92 of the reference
    torch.manual_seed(3)
    w = torch.randn(128, 256)
    ip = qtip.IPContext(w, cb_rms=1.0, seed=0)
    assert torch.allclose(ip.restore(ip.z), w, atol=1e-5)
    assert abs(float(ip.z.square().mean().sqrt()) - 1.0) < 1e-4
    odd = torch.randn(48, 576)                     # 576 = 64 * 9: block shrinks to the largest power-of-two divisor
    ip2 = qtip.IPContext(odd, cb_rms=1.0, seed=1)
    assert torch.allclose(ip2.restore(ip2.z), odd, atol=1e-5)


def test_block_ldl_identity_and_structure():
    # tests/test_ldlq.py:12-17
    L0 = ldlq.block_ldl(ldlq.regularize_H(torch.eye(64), 0.0), b=16)
    assert torch.allclose(L0, torch.zeros_like(L0), atol=1e-6)
    torch.manual_seed(0)
    A = torch.randn(64, 64)
    H = A.T @ A / 64 + torch.eye(64)
    Lm = ldlq.block_ldl(H, b=16)
    for i in range(4):                                                     # diagonal blocks: unit lower triangular minus I
        blk = Lm[16 * i:16 * i + 16, 16 * i:16 * i + 16]
        assert torch.allclose(blk, torch.zeros_like(blk), atol=1e-5)
    assert float(torch.triu(Lm, 1).abs().max()) == 0.0
    assert ldlq.block_ldl(torch.full((32, 32), float("nan")), b=16) is None


def test_ldlq_recursion_with_a_stand_in_quantizer():
    """With enc = round-to-grid the recursion must satisfy its defining fixed point:
    every block is the quantisation of (W + L^T (W - Wq)) restricted to later rows."""
    torch.manual_seed(1)
    k, n = 256, 32
    Wt = torch.randn(k, n)
    A = torch.randn(k, k)
    Lm = ldlq.block_ldl(A.T @ A / k + torch.eye(k), b=16)
    enc = lambda rows: torch.round(rows * 4) / 4
    for buf in (128, 64):
        Wq = ldlq.ldlq(Wt, Lm, enc, buf=buf)
        target = Wt + Lm.t() @ (Wt - Wq)
        assert torch.allclose(Wq, enc(target), atol=0.2501)       # equal up to rounding-boundary flips ...
        assert float((Wq != enc(target)).float().mean()) < 0.01   # ... which are rare
    calls = []
    ldlq.ldlq(Wt, torch.zeros(k, k), lambda r: (calls.append(r.clone()), r)[1])
    assert len(calls) == k // 16 and torch.equal(calls[0], Wt[k - 16:])   # reverse order, raw targets when L = 0


def test_row_block_tiles():
    rows = torch.arange(16 * 64, dtype=torch.float32).reshape(16, 64)
    tiles = ldlq.rows_to_tiles(rows)
    assert tiles.shape == (4, 256)
    assert tiles[2, 5 * 16 + 3] == rows[3, 2 * 16 + 5]            # t = (out % 16) * 16 + in
    assert torch.equal(ldlq.tiles_to_rows(tiles, 64), rows)


def test_tile_ranges_and_matrix_assignment():
    for n, world in ((10, 4), (65536, 8), (3, 8), (0, 2)):
        spans = [tdist.tile_range(n, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert max(b - a for a, b in spans) - min(b - a for a, b in spans) <= 1
    plan = tdist.assign_matrices([5, 3, 3, 2, 2, 1], 2)
    assert sorted(i for p in plan for i in p) == list(range(6))
    assert abs(sum([5, 3, 3, 2, 2, 1][i] for i in plan[0]) - 8) <= 1
    shapes = {f"l{i}.{m}": s for i in range(2) for m, s in (("q", (4096, 4096)), ("down", (4096, 12288)))}
    names = tdist.model_plan(shapes, [n for n in shapes if "down" in n], 2)
    assert sorted(sum(names, [])) == sorted(shapes)


def _gloo_worker(rank, world, port, n_total, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as O                      # CPU stand-in for the encoder, tests only
        rng = np.random.default_rng(0)
        w = rng.standard_normal((n_total, 256)).astype(np.float32)
        lut = O.codebook_lut("mcg")

        def cpu_encoder(tiles, K, codebook):
            bits, dq = O.viterbi_tb(tiles.numpy(), K, lut, nthreads=1)
            packed = torch.from_numpy(O.pack_bits(bits, K).view(np.int32))
            return qtip.Encoded(packed, torch.from_numpy(dq), None, torch.from_numpy(bits))

        every, local, (lo, hi) = tdist.encode_sharded(torch.from_numpy(w), 3, "mcg", encoder=cpu_encoder)
        only0, _, _ = tdist.encode_sharded(torch.from_numpy(w), 3, "mcg", dst=0, encoder=cpu_encoder)
        assert (only0 is None) == (rank != 0)
        assert local.packed.shape[0] == hi - lo
        torch.save({"all": every, "dst0": only0}, os.path.join(tmp, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_two_rank_shard_and_gather_over_gloo(tmp_path, oracle, luts):
    n_total, world = 5, 2                                    # ragged: 3 + 2 tiles
    port = 29500 + os.getpid() % 2000
    mp.start_processes(_gloo_worker, args=(world, port, n_total, str(tmp_path)), nprocs=world, join=True,
                       start_method="spawn")
    rng = np.random.default_rng(0)
    w = rng.standard_normal((n_total, 256)).astype(np.float32)
    bits, _ = oracle.viterbi_tb(w, 3, luts["mcg"])
    want = oracle.pack_bits(bits, 3).view(np.int32)
    r0 = torch.load(os.path.join(tmp_path, "r0.pt"))
    r1 = torch.load(os.path.join(tmp_path, "r1.pt"))
    assert np.array_equal(r0["all"].numpy(), want) and np.array_equal(r1["all"].numpy(), want)
    assert np.array_equal(r0["dst0"].numpy(), want) and r1["dst0"] is None


def _gloo_model_gather_worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from trellis_b200 import model
        shapes = {f"model.layers.{i}.{m}": s for i in range(2)
                  for m, s in (("self_attn.q_proj", (32, 64)), ("mlp.up_proj", (96, 32)), ("mlp.down_proj", (32, 96)))}
        ldlq_names = [n for n in shapes if model.is_mlp(n)]
        mine = tdist.model_plan(shapes, ldlq_names, world)[rank]
        # stand-in code words: a pattern that encodes (matrix, tile, word) so misplaced rows are caught
        names = sorted(shapes)
        fake = lambda n: (torch.arange((shapes[n][0] // 16) * (shapes[n][1] // 16) * 24, dtype=torch.int32).reshape(-1, 24)
                          + 100000 * names.index(n))
        got = model.gather_model_codes(shapes, ldlq_names, {n: fake(n) for n in mine}, 3, world, rank, torch.device("cpu"))
        if rank == 0:
            assert set(got) == set(shapes)
            assert all(torch.equal(got[n], fake(n)) for n in shapes)
            open(os.path.join(tmp, "ok"), "w").write("ok")
        else:
            assert got is None
    finally:
        dist.destroy_process_group()


def test_model_code_gather_over_gloo(tmp_path):
    port = 31500 + os.getpid() % 2000
    mp.start_processes(_gloo_model_gather_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True, start_method="spawn")
    assert os.path.exists(os.path.join(tmp_path, "ok"))


def test_shard_writer_reproduces_the_reference_shard_byte_for_byte(tmp_path, golden):
    """A shard written here from the same packed words and incoherence-processing vectors is the reference
    exporter's file: identical .bin bytes and identical .bin.json index (scripts/export_packed_8b.py:65-79,134-143)."""
    import json
    import types
    from trellis_b200 import shards
    g = golden["shard"]
    name = bytes(g["name"]).decode()
    n, k = g["w"].shape
    K = int(g["K"])
    ip = types.SimpleNamespace(su=torch.from_numpy(g["su"]), sv=torch.from_numpy(g["sv"]), in_s=torch.from_numpy(g["in_s"]),
                               out_s=torch.from_numpy(g["out_s"]), scale=float(g["scale"]))
    path = str(tmp_path / "layer_00.bin")
    assert not shards.shard_done(path)
    sh = shards.Shard(path)
    sh.put_quant(name, torch.from_numpy(g["packed"].view(np.int32)), ip, n, k, K)     # int32 words, as the GPU returns them
    sh.put("model.layers.0.input_layernorm.weight", g["norm"], np.float16)
    with pytest.raises(KeyError):
        sh.put(name + ".bits", g["packed"], np.uint32)
    with pytest.raises(ValueError):
        sh.put("bad", g["norm"], np.float64)
    sh.flush()
    assert shards.shard_done(path)
    assert np.array_equal(np.fromfile(path, dtype=np.uint8), g["bin"])
    assert json.load(open(path + ".json")) == json.loads(bytes(g["index"]).decode())

    man = shards.merge_manifest(str(tmp_path))
    assert json.load(open(tmp_path / "manifest.json")) == man
    q = shards.read_quant(str(tmp_path), man, name)
    assert q["n_out"] == n and q["k_in"] == k and q["K"] == K and q["tiles_in"] == k // 16 and q["block"] == 64
    assert np.array_equal(q["bits"], g["packed"]) and q["bits"].dtype == np.uint32
    assert np.array_equal(q["su"].astype(np.float32), g["su"]) and np.array_equal(q["osc"], g["out_s"].astype(np.float16))
    assert np.array_equal(shards.read_tensor(str(tmp_path), man, "model.layers.0.input_layernorm.weight"), g["norm"].astype(np.float16))
    with pytest.raises(KeyError):
        shards.read_tensor(str(tmp_path), man, name)

    # the mirror's incoherence processing gives the same vectors as the reference's (same generator, same recipe)
    mine = qtip.IPContext(torch.from_numpy(g["w"]), _mcg_rms(), seed=zlib.crc32(b"x"))
    assert torch.equal(mine.su, ip.su) and torch.equal(mine.sv, ip.sv)
    assert torch.allclose(mine.in_s, ip.in_s, rtol=1e-5) and torch.allclose(mine.out_s, ip.out_s, rtol=1e-5)
    assert abs(mine.scale - ip.scale) < 1e-5 * ip.scale


def _mcg_rms() -> float:
    """RMS of the MCG codebook, computed on the host from its definition (qtip.py:51-56)."""
    s = np.arange(65536, dtype=np.uint64)
    v = (s * np.uint64(0xCBAC1FED)) & np.uint64(0xFFFFFFFF)
    r = ((v & np.uint64(0x8FFF8FFF)) ^ np.uint64(0x3B603B60)).astype(np.uint32)
    hi = (r >> np.uint32(16)).astype(np.uint16).view(np.float16).astype(np.float32)
    lo = (r & np.uint32(0xFFFF)).astype(np.uint16).view(np.float16).astype(np.float32)
    return float(torch.from_numpy(hi + lo).square().mean().sqrt().item())


def test_model_shapes_match_the_fifth_configuration():
    """252 linears / 6 945 767 424 weights / 27 131 904 tiles of the Qwen3-8B shape that the reference's loop walks
    (scripts/run_tcq_eval.py:106-127), plus the two embedding-sized matrices its exporter packs on request."""
    from trellis_b200 import model
    shapes = model.qwen3_8b_shapes()
    assert len(shapes) == 252
    assert sum(n * k for n, k in shapes.values()) == 6_945_767_424
    assert sum((n // 16) * (k // 16) for n, k in shapes.values()) == 27_131_904
    assert sum(model.is_mlp(n) for n in shapes) == 108
    more = model.qwen3_8b_shapes(embeddings=True)
    assert len(more) == 254 and more["lm_head"] == (151936, 4096) == more["model.embed_tokens"]
    plan = tdist.model_plan(more, [n for n in more if model.is_mlp(n)], 8)
    assert sorted(n for p in plan for n in p) == sorted(more)
    assert {plan[0][0], plan[1][0]} == {"lm_head", "model.embed_tokens"}        # the two largest go first, on different ranks
    assert model.seed_of("model.layers.0.mlp.up_proj") == __import__("zlib").crc32(b"model.layers.0.mlp.up_proj")


def _gloo_leaver_worker(rank, world, port, tmp):
    """Rank 1 leaves between steps, before the gather; rank 0 must get a clean error within seconds, not hang."""
    import datetime
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    local = torch.arange(3 * 24, dtype=torch.int32).reshape(3, 24) if rank == 0 else torch.zeros((2, 24), dtype=torch.int32)
    dist.barrier()                                           # both ranks are up; the rendezvous worked
    if rank == 1:
        os._exit(0)                                          # dies with nothing in flight
    t0 = time.monotonic()
    try:
        tdist.gather_packed(local, 5, dst=0)
        outcome = "returned"
    except Exception as e:                                   # gloo reports the lost peer or the timeout
        outcome = "error:" + type(e).__name__
    open(os.path.join(tmp, "r0"), "w").write(f"{outcome} {time.monotonic() - t0:.1f}")
    os._exit(0)                                              # the group is broken: no orderly teardown to wait for


def test_gather_fails_cleanly_when_a_rank_has_left(tmp_path):
    """Host-side failure detection of the one collective: a rank that exits before ``gather_packed`` turns into an
    exception on the surviving rank within the process group's timeout."""
    port = 33500 + os.getpid() % 2000
    ctx = mp.start_processes(_gloo_leaver_worker, args=(2, port, str(tmp_path)), nprocs=2, join=False, start_method="spawn")
    import time
    deadline = time.monotonic() + 60
    while not os.path.exists(os.path.join(tmp_path, "r0")) and time.monotonic() < deadline:
        time.sleep(0.2)
    for p in ctx.processes:
        p.join(timeout=10)
        if p.is_alive():
            p.kill()
    outcome, secs = open(os.path.join(tmp_path, "r0")).read().split()
    assert outcome.startswith("error:"), outcome
    assert float(secs) < 30


def test_second_configuration_tiles_agree_with_the_reference(golden, oracle, luts):
    """``workloads.cfg2_tiles`` (CPU generator + the host form of incoherence processing) against 16 tiles of the
    same matrix as the reference's own ``IPContext`` produced them."""
    from trellis_b200 import workloads
    g = golden["cfg2_probe"]
    tiles = workloads.cfg2_tiles(torch.from_numpy(luts["3inst"]))
    assert tiles.shape == (65536, 256) and tiles.dtype == torch.float32
    mine = tiles[torch.from_numpy(g["index"])].numpy()
    assert np.allclose(mine, g["tiles"], rtol=0, atol=2e-5)
    assert abs(float(tiles.square().mean().sqrt()) - float(g["z_rms"])) < 1e-4


def test_resume_ignores_stale_or_foreign_files(tmp_path):
    """The resume check of ``encode_model`` is pure host logic: exercised here with a stand-in for the encoder."""
    from trellis_b200 import model
    import json
    shapes = {"model.layers.0.self_attn.k_proj": (32, 64)}
    calls = []

    def fake_encode_matrix(w, K, codebook, seed, H=None, return_ip=False, **kw):
        calls.append((K, seed))
        n, k = w.shape
        packed = torch.full(((n // 16) * (k // 16), 8 * K), len(calls), dtype=torch.int32)
        return packed, w, 0.0, None

    real = model.encode_matrix, model.qtip.workspace_status, model.qtip.codebook_id
    model.encode_matrix = fake_encode_matrix
    model.qtip.workspace_status = lambda *a, **k: None

    class _S:
        def synchronize(self):
            pass

    try:
        import unittest.mock as um
        with um.patch.object(torch.cuda, "current_stream", lambda dev=None: _S()), \
                um.patch.object(torch.cuda, "current_device", lambda: 0):
            run = lambda **kw: model.encode_model(shapes, hessian_fn=None, weight_fn=lambda n, s, d: torch.zeros(s), out_dir=str(tmp_path),
                                                  device=torch.device("cpu"), gather=False, **kw)
            r1, _ = run(K=3, codebook="mcg")
            assert not r1["model.layers.0.self_attn.k_proj"]["skipped"] and len(calls) == 1
            r2, _ = run(K=3, codebook="mcg")
            assert r2["model.layers.0.self_attn.k_proj"]["skipped"] and len(calls) == 1          # same settings: resumed
            r3, _ = run(K=4, codebook="mcg")
            assert not r3["model.layers.0.self_attn.k_proj"]["skipped"] and len(calls) == 2      # other K: encoded again
            r4, _ = run(K=4, codebook="3inst")
            assert not r4["model.layers.0.self_attn.k_proj"]["skipped"] and len(calls) == 3      # other codebook
            r5, _ = run(K=4, codebook="3inst", seed_fn=lambda n: 7)
            assert not r5["model.layers.0.self_attn.k_proj"]["skipped"] and len(calls) == 4      # other seed
            meta = json.load(open(os.path.join(tmp_path, "model.layers.0.self_attn.k_proj.bits.npy.json")))
            assert meta == {"K": 4, "codebook": "3inst", "shape": [32, 64], "seed": 7, "ldlq": False}
            os.remove(os.path.join(tmp_path, "model.layers.0.self_attn.k_proj.bits.npy.json"))
            r6, _ = run(K=4, codebook="3inst", seed_fn=lambda n: 7)
            assert not r6["model.layers.0.self_attn.k_proj"]["skipped"]                          # no side-car: not trusted
    finally:
        model.encode_matrix, model.qtip.workspace_status, model.qtip.codebook_id = real


def test_reference_staging_recipe(tmp_path, monkeypatch):
    """oracle/make_ref.py: what it stages is byte-identical to the checkout (digest check), a tampered copy is not
    accepted, and without a checkout it stages nothing.  Skipped where no checkout of the reference is at hand."""
    import hashlib
    import shutil
    from oracle import make_ref
    assert make_ref.stage(str(tmp_path / "no_such_checkout")) is None
    src = os.path.join(make_ref.default_checkout(), "src", "trellis")
    if not all(os.path.isfile(os.path.join(src, f)) for f in make_ref.FILES):
        pytest.skip("no checkout of the reference here")
    monkeypatch.setattr(make_ref, "REF_DIR", str(tmp_path / "_ref"))
    assert make_ref.staged() is None
    assert make_ref.stage() == str(tmp_path / "_ref") and make_ref.staged() == str(tmp_path / "_ref")
    for f in make_ref.FILES:
        a = hashlib.sha256(open(os.path.join(src, f), "rb").read()).hexdigest()
        b = hashlib.sha256(open(os.path.join(tmp_path, "_ref", "trellis", f), "rb").read()).hexdigest()
        assert a == b
    with open(os.path.join(tmp_path, "_ref", "trellis", "qtip.py"), "a") as fh:
        fh.write("# edited\n")
    assert make_ref.staged() is None                       # a modified copy is not "the reference"
    shutil.rmtree(tmp_path / "_ref")


def test_row_block_wrapper_rejects_bad_arguments_before_touching_the_gpu():
    """``qtip.encode_rows`` validates shapes, strides and devices on the host; none of these reach the library."""
    z = torch.zeros(16, 64)
    with pytest.raises(ValueError, match="16, n_out"):
        qtip.encode_rows(torch.zeros(8, 64), None, 3, "mcg", torch.zeros(8, 64))
    with pytest.raises(ValueError, match="n_out % 16"):
        qtip.encode_rows(torch.zeros(16, 40), None, 3, "mcg", torch.zeros(16, 40))
    with pytest.raises(ValueError, match="K must be"):
        qtip.encode_rows(z, None, 5, "mcg", torch.zeros(16, 64))
    with pytest.raises(ValueError, match="unknown codebook"):
        qtip.encode_rows(z, None, 3, "nope", torch.zeros(16, 64))
    with pytest.raises(ValueError, match="CUDA tensors only"):
        qtip.encode_rows(z, None, 3, "mcg", torch.zeros(16, 64))
