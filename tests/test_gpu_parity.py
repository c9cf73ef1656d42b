"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle.

Bit-exact for the lattice decode; for the GEMV the tolerances the benchmark specification states:
relative L2 <= 1e-5 with f32 activations, <= 1e-3 with f16 activations, plus the
reference's own per-row criterion max |got - ref| / sum |w_i x_i| < 1e-5 for f32
(llvq-cuda/src/bin/matvec.rs:63,114-120).
"""
import ctypes as C

import numpy as np
import pytest

from conftest import probe_indices

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-5
TOL_F16 = 1e-3


def rel_l2(got, ref):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    return float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-300))


def _torch():
    import torch
    return torch


def gpu_gemv(rt, m, x, mode="same", tail_f16=False):
    torch = _torch()
    proj = rt.upload(m, tail_f16=tail_f16)
    xd = torch.from_numpy(x).cuda()
    y = rt.forward_rotated(proj, xd) if mode == "f32x_h" else rt.forward(proj, xd)
    torch.cuda.synchronize()
    out = y.cpu().numpy()
    proj.free()
    return out


def test_runtime_reproduces_published_fingerprint(rt, oracle):
    assert rt.fingerprint() == oracle.PUBLISHED_FINGERPRINT
    assert rt.codebook_info(12) == (301, oracle.N12)
    assert rt.codebook_info(13) == (383, oracle.N13)


def test_decode_indices_every_class_boundary(rt, oracle):
    torch = _torch()
    idx = probe_indices(oracle, per_class_random=50, cap=13)
    pts, shell = rt.decode_indices(torch.from_numpy(idx.view(np.int64)).cuda())
    pts, shell = pts.cpu().numpy(), shell.cpu().numpy()
    for k, i in enumerate(idx):
        assert np.array_equal(pts[k], oracle.decode_index(int(i), 13)), int(i)
    extra = np.array([oracle.N13, oracle.N13 + 1, (1 << 48) - 1, 1 << 63], np.uint64)
    pts, shell = rt.decode_indices(torch.from_numpy(extra.view(np.int64)).cuda())
    assert shell.cpu().tolist() == [13, 255, 255, 255] and not pts[1:].cpu().numpy().any()


def test_decode_blocks_bit_exact_on_uniform_draws(rt, oracle):
    torch = _torch()
    from llvq_b200 import synth
    g = synth.SplitMix64(0xB10C)
    n = 2_000_000
    idx = g.take(n) % np.uint64(oracle.N12 + 1)
    gain = g.take(n) & np.uint64(1)
    codes = synth.pack_codes(idx, gain)
    pts, shell, gn = rt.decode_blocks(torch.from_numpy(codes).cuda())
    ref_pts, ref_shell, ref_gain, bad = oracle.decode_codes(codes)
    assert bad == 0
    assert np.array_equal(pts.cpu().numpy(), ref_pts)
    assert np.array_equal(shell.cpu().numpy(), ref_shell)
    assert np.array_equal(gn.cpu().numpy(), ref_gain)


def test_decode_blocks_edge_records(rt, oracle):
    torch = _torch()
    from llvq_b200 import synth
    idx = np.concatenate([probe_indices(oracle, cap=12), np.array([oracle.N12 + 1, (1 << 47) - 1], np.uint64)])
    gain = (np.arange(idx.size) & 1).astype(np.uint64)
    codes = synth.pack_codes(idx, gain)
    pts, shell, gn = rt.decode_blocks(torch.from_numpy(codes).cuda())
    ref_pts, ref_shell, ref_gain, bad = oracle.decode_codes(codes, use_ref=True)
    assert bad == 2
    assert np.array_equal(pts.cpu().numpy(), ref_pts)
    assert np.array_equal(shell.cpu().numpy(), ref_shell) and shell[-1].item() == 255
    assert np.array_equal(gn.cpu().numpy(), ref_gain)
    # empty input is a no-op, even with null pointers
    e_pts, e_shell, e_gain = rt.decode_blocks(torch.empty(0, dtype=torch.uint8, device="cuda"))
    assert e_pts.shape == (0, 24)


def test_fused_kernel_decoders_bit_exact_on_every_class(rt, oracle):
    """The decoders the GEMV and GEMM kernels run (class search + family decoders, tables in shared memory),
    dumped on the device: both ends of all 301 classes, their neighbours, 200 draws inside each class."""
    torch = _torch()
    from llvq_b200 import synth
    idx = np.concatenate([probe_indices(oracle, per_class_random=200, cap=12),
                          np.array([oracle.N12 + 1, (1 << 47) - 1], np.uint64)])
    gain = (np.arange(idx.size) & 1).astype(np.uint64)
    codes = synth.pack_codes(idx, gain)
    pts, shell, gn = rt.decode_blocks_fast(torch.from_numpy(codes).cuda())
    ref_pts, ref_shell, ref_gain, bad = oracle.decode_codes(codes, use_ref=True)
    assert bad == 2
    assert np.array_equal(pts.cpu().numpy(), ref_pts)
    assert np.array_equal(shell.cpu().numpy(), ref_shell) and shell[-1].item() == 255
    assert np.array_equal(gn.cpu().numpy(), ref_gain)
    e_pts, _, _ = rt.decode_blocks_fast(torch.empty(0, dtype=torch.uint8, device="cuda"))
    assert e_pts.shape == (0, 24)


def test_fused_kernel_decoders_bit_exact_on_ten_million_draws(rt, oracle):
    torch = _torch()
    from llvq_b200 import synth
    g = synth.SplitMix64(0xFA57B10C)
    n = 10_000_000
    idx = g.take(n) % np.uint64(oracle.N12 + 1)
    gain = g.take(n) & np.uint64(1)
    codes = synth.pack_codes(idx, gain)
    pts, shell, gn = rt.decode_blocks_fast(torch.from_numpy(codes).cuda())
    # the generic device decoder is pinned to the oracle by the tests above; the oracle itself checks a slice
    ref_pts, ref_shell, ref_gn = rt.decode_blocks(torch.from_numpy(codes).cuda())
    assert torch.equal(pts, ref_pts) and torch.equal(shell, ref_shell) and torch.equal(gn, ref_gn)
    k = 500_000
    o_pts, o_shell, o_gain, bad = oracle.decode_codes(codes[:6 * k])
    assert bad == 0 and np.array_equal(pts[:k].cpu().numpy(), o_pts) and np.array_equal(shell[:k].cpu().numpy(), o_shell)


@pytest.mark.parametrize("d_out,d_in", [(8, 24), (16, 127), (9, 24 * 7 + 3), (1, 48), (40, 23), (64, 2560), (24, 9728)])
def test_gemv_f32_small_and_ragged(rt, oracle, d_out, d_in):
    from llvq_b200 import synth
    m = synth.make_matrix(d_out, d_in, 1000 + d_out * 7 + d_in)
    x = synth.make_activation(d_in, 77 + d_in)
    y = gpu_gemv(rt, m, x)
    ref, absdot = oracle.gemv_f64(m.codes, d_out, d_in, m.centroids, m.row_scales, m.tail, x.astype(np.float64),
                                  use_ref=True, want_absdot=True)
    assert rel_l2(y, ref) <= TOL_F32
    assert np.max(np.abs(y - ref) / np.maximum(absdot, 1e-300)) < 1e-5


def test_gemv_config0_up_proj_f32(rt, oracle):
    """benchmark configuration 0: W 9728 x 2560 (106 blocks + 16 tail columns), f32 activation."""
    from llvq_b200 import synth
    m = synth.make_matrix(9728, 2560, synth.matrix_seed(0, 0, synth.PROJ_IDS["up"]), "up")
    x = synth.make_activation(2560, synth.matrix_seed(0, 0, 5))
    y = gpu_gemv(rt, m, x)
    ref, absdot = oracle.gemv_f64(m.codes, m.d_out, m.d_in, m.centroids, m.row_scales, m.tail, x.astype(np.float64),
                                  want_absdot=True)
    assert rel_l2(y, ref) <= TOL_F32
    assert np.max(np.abs(y - ref) / absdot) < 1e-5
    assert not rt.poll_range_error()


def test_gemv_config1_layer_f16(rt, oracle):
    """benchmark configuration 1: the seven projections of one Qwen3-4B layer, f16 activations and results."""
    from llvq_b200 import synth
    layer = synth.make_layer("qwen3-4b", 1, 0)
    for name, m in layer.items():
        x = synth.make_activation(m.d_in, synth.matrix_seed(1, 0, synth.PROJ_IDS[name]), np.float16)
        y = gpu_gemv(rt, m, x, tail_f16=True)
        tail16 = m.tail.astype(np.float16).astype(np.float32)
        ref = oracle.gemv_f64(m.codes, m.d_out, m.d_in, m.centroids, m.row_scales, tail16, x.astype(np.float64))
        assert y.dtype == np.float16
        assert rel_l2(y, ref) <= TOL_F16, name


def test_gemv_f32x_h_matches_reference_signature(rt, oracle):
    from llvq_b200 import synth
    m = synth.make_matrix(1024, 2560, 31337)
    x = synth.make_activation(2560, 4242)
    y = gpu_gemv(rt, m, x, mode="f32x_h", tail_f16=True)
    tail16 = m.tail.astype(np.float16).astype(np.float32)
    ref = oracle.gemv_f64(m.codes, m.d_out, m.d_in, m.centroids, m.row_scales, tail16, x.astype(np.float64))
    assert y.dtype == np.float16 and rel_l2(y, ref) <= TOL_F16


def test_group_upload_equals_separate_projections(rt, oracle):
    torch = _torch()
    from llvq_b200 import synth
    parts = [synth.make_matrix(d, 24 * 20 + 8, 900 + i) for i, d in enumerate((64, 16, 24))]
    x = synth.make_activation(parts[0].d_in, 5)
    xd = torch.from_numpy(x).cuda()
    grp = rt.upload_group(parts)
    assert grp.d_out == 104 and grp.splits == [64, 16, 24]
    yg = rt.forward(grp, xd).cpu().numpy()
    ys = np.concatenate([gpu_gemv(rt, p, x) for p in parts])
    assert np.array_equal(yg, ys)  # same kernel, same rows: identical bits
    ref = np.concatenate([oracle.gemv_f64(p.codes, p.d_out, p.d_in, p.centroids, p.row_scales, p.tail, x.astype(np.float64))
                          for p in parts])
    assert rel_l2(yg, ref) <= TOL_F32


def test_output_buffer_is_fully_overwritten(rt):
    torch = _torch()
    from llvq_b200 import synth
    m = synth.make_matrix(72, 24 * 9, 11)
    proj = rt.upload(m)
    xd = torch.from_numpy(synth.make_activation(m.d_in, 3)).cuda()
    a = rt.forward(proj, xd, out=torch.full((72,), float("nan"), device="cuda"))
    b = rt.forward(proj, xd, out=torch.full((72,), 1e30, device="cuda"))
    assert torch.isfinite(a).all() and torch.equal(a, b)


def test_linearity_at_full_size(rt):
    """Size-independent property on the 9728 x 2560 shape: W(a x1 + x2) = a W x1 + W x2 within f32 rounding."""
    torch = _torch()
    from llvq_b200 import synth
    m = synth.make_matrix(9728, 2560, 123456)
    proj = rt.upload(m)
    x1 = torch.from_numpy(synth.make_activation(2560, 1)).cuda()
    x2 = torch.from_numpy(synth.make_activation(2560, 2)).cuda()
    y1, y2 = rt.forward(proj, x1).double(), rt.forward(proj, x2).double()
    y12 = rt.forward(proj, 0.5 * x1 + x2).double()
    err = (y12 - (0.5 * y1 + y2)).norm() / y12.norm()
    assert err.item() < 1e-5
    z = rt.forward(proj, torch.zeros(2560, device="cuda"))
    assert not z.any()


def test_host_buffer_entry_point(rt, oracle):
    from llvq_b200 import synth
    m = synth.make_matrix(128, 24 * 30 + 4, 2024)
    proj = rt.upload(m)
    for dt, tol in ((np.float32, TOL_F32), (np.float16, TOL_F16)):
        x = synth.make_activation(m.d_in, 9, dt)
        y = np.empty(m.d_out, dt)
        rt.forward_host(proj, x, y)
        ref = oracle.gemv_f64(m.codes, m.d_out, m.d_in, m.centroids, m.row_scales, m.tail, x.astype(np.float64))
        assert rel_l2(y, ref) <= tol


def test_host_buffer_list_entry_point(rt, oracle):
    from llvq_b200 import synth
    ms = [synth.make_matrix(d, 24 * 12 + 3, 600 + d) for d in (64, 8, 40)]
    projs = [rt.upload(m, tail_f16=True) for m in ms]
    xs = [synth.make_activation(m.d_in, 70 + i, np.float16) for i, m in enumerate(ms)]
    ys = [np.full(m.d_out, np.nan, np.float16) for m in ms]
    rt.forward_host_many(projs, xs, ys)
    singles = []
    for m, p, x, y in zip(ms, projs, xs, ys):
        single = np.empty(m.d_out, np.float16)
        rt.forward_host(p, x, single)
        assert np.array_equal(y, single)
        singles.append(single)
    rt.forward_host_many([], [], [])
    # the list travels in up to eight segments (short ones at both ends from 64 calls on): every length around the
    # switches gives every call its own result, twice in a row on the same staging buffers
    for n in (1, 2, 7, 8, 9, 31, 63, 64, 65, 100, 257):
        order = [(7 * i + n) % 3 for i in range(n)]
        ys_n = [np.full(ms[k].d_out, np.nan, np.float16) for k in order]
        for _ in range(2):
            rt.forward_host_many([projs[k] for k in order], [xs[k] for k in order], ys_n)
            for k, y in zip(order, ys_n):
                assert np.array_equal(y, singles[k]), (n, k)


def test_index_outside_the_ball_raises_the_range_flag(rt, oracle):
    torch = _torch()
    from llvq_b200 import synth
    m = synth.make_matrix(8, 48, 5)
    idx, gain = synth.unpack_codes(m.codes)
    idx[3] = oracle.N12 + 5
    m.codes = synth.pack_codes(idx, gain)
    proj = rt.upload(m)
    assert not rt.poll_range_error()
    y = rt.forward(proj, torch.ones(48, device="cuda"))
    assert rt.poll_range_error() and not rt.poll_range_error()  # sticky until polled, then cleared
    assert torch.isfinite(y).all()  # the refused block contributes zero; nothing traps


def test_argument_errors_are_statuses_not_crashes(rt):
    torch = _torch()
    from llvq_b200 import LlvqError, _lib, synth
    m = synth.make_matrix(8, 48, 1)
    m.shell_cap = 13
    with pytest.raises(LlvqError) as e:
        rt.upload(m)
    assert e.value.status == _lib.ERR_UNSUPPORTED and "cap" in e.value.message
    m.shell_cap = 12
    m.centroids = np.array([1.0, 2.0, 3.0])
    with pytest.raises(ValueError):
        rt.upload(m)
    m.centroids = np.array([1.0, 2.0])
    proj = rt.upload(m)
    with pytest.raises(ValueError):
        rt.forward(proj, torch.ones(47, device="cuda"))
    with pytest.raises(ValueError):
        rt.forward(proj, torch.ones(96, device="cuda")[::2])
    with pytest.raises(TypeError):
        rt.forward(proj, torch.ones(48, device="cuda", dtype=torch.bfloat16))
    L = _lib.load()
    assert L.llvq_gemv_f32(proj._h, C.c_void_p(2), C.c_void_p(4), None) == _lib.ERR_INVALID  # misaligned
    h = C.c_void_p()
    assert L.llvq_runtime_create(99, C.byref(h)) == _lib.ERR_INVALID


def test_batch_forward_matches_row_by_row(rt, oracle):
    torch = _torch()
    from llvq_b200 import synth
    m = synth.make_matrix(256, 24 * 40 + 16, 77)
    proj = rt.upload(m, tail_f16=True)
    for batch in (1, 3, 16, 64):
        x = synth.make_activation(m.d_in, 500 + batch, np.float16, batch=batch)
        y = rt.forward_batch(proj, torch.from_numpy(x).cuda()).cpu().numpy()
        tail16 = m.tail.astype(np.float16).astype(np.float32)
        ref = oracle.gemv_f64(m.codes, m.d_out, m.d_in, m.centroids, m.row_scales, tail16, x.astype(np.float64))
        assert y.shape == (batch, 256) and rel_l2(y, ref) <= TOL_F16


@pytest.mark.parametrize("d_out,d_in,batch", [(128, 192, 16), (200, 24 * 11 + 5, 17), (384, 24 * 19, 32), (136, 24 * 8 + 12, 100),
                                              (72, 30, 16)])
def test_batched_gemm_ragged_shapes(rt, oracle, d_out, d_in, batch):
    """tcgen05 path: row tiles, column chunks, batch padding and the unaligned-x route all have ragged cases."""
    torch = _torch()
    from llvq_b200 import synth
    m = synth.make_matrix(d_out, d_in, 0x6E44 + d_out + d_in)
    proj = rt.upload(m, tail_f16=True)
    x = synth.make_activation(d_in, 0x77 + batch, np.float16, batch=batch)
    y = rt.forward_batch(proj, torch.from_numpy(x).cuda()).cpu().numpy()
    tail16 = m.tail.astype(np.float16).astype(np.float32)
    ref = oracle.gemv_f64(m.codes, d_out, d_in, m.centroids, m.row_scales, tail16, x.astype(np.float64))
    assert y.shape == (batch, d_out) and np.isfinite(y).all()
    assert rel_l2(y, ref) <= TOL_F16
    for n in (0, batch - 1):  # every batch row on its own, not just the aggregate
        assert rel_l2(y[n], ref[n]) <= 2 * TOL_F16
    assert not rt.poll_range_error()


def test_batched_gemm_config3_qwen3_8b_shapes(rt, oracle):
    """benchmark configuration 3: tree-verify batches of 16 and 64 on Qwen3-8B shapes (k_proj and a slice of gate_proj)."""
    torch = _torch()
    from llvq_b200 import synth
    for d_out, d_in in ((1024, 4096), (1536, 4096), (512, 12288)):
        m = synth.make_matrix(d_out, d_in, synth.matrix_seed(3, 0, d_out % 7))
        proj = rt.upload(m, tail_f16=True)
        tail16 = m.tail.astype(np.float16).astype(np.float32)
        for batch in (16, 64):
            x = synth.make_activation(d_in, 0x300 + batch, np.float16, batch=batch)
            y = rt.forward_batch(proj, torch.from_numpy(x).cuda()).cpu().numpy()
            ref = oracle.gemv_f64(m.codes, d_out, d_in, m.centroids, m.row_scales, tail16, x.astype(np.float64))
            assert rel_l2(y, ref) <= TOL_F16, (d_out, d_in, batch)
        proj.free()


def test_batched_gemm_equals_gemv_semantics(rt):
    """The same activation in every batch row gives the same output row, close to the batch-1 kernel's."""
    torch = _torch()
    from llvq_b200 import synth
    m = synth.make_matrix(256, 24 * 64, 4711)
    proj = rt.upload(m, tail_f16=True)
    x1 = torch.from_numpy(synth.make_activation(m.d_in, 5, np.float16)).cuda()
    yb = rt.forward_batch(proj, x1.repeat(16, 1).contiguous())
    assert torch.equal(yb[0], yb[15])
    y1 = rt.forward(proj, x1).float()
    assert ((yb[0].float() - y1).norm() / y1.norm()).item() < 2e-3


@pytest.mark.parametrize("d_out,d_in", [(40, 24 * 7 + 5), (64, 24 * 16), (17, 30), (8, 12)])
def test_dense_dequant_matches_the_oracle_matrix(rt, oracle, d_out, d_in):
    """llvq_matrix_dequant_h writes f16(oracle weight): same lattice points, gain, row scale and tail."""
    torch = _torch()
    from llvq_b200 import synth
    m = synth.make_matrix(d_out, d_in, 0xDE45E + d_out)
    proj = rt.upload(m, tail_f16=True)
    w = rt.dequant(proj).cpu().numpy().astype(np.float64)
    tail16 = m.tail.astype(np.float16).astype(np.float32)
    want = oracle.decode_matrix(m.codes, d_out, d_in, m.centroids, m.row_scales, tail16).astype(np.float64)
    assert w.shape == want.shape
    # one f16 rounding of a product formed in f32: 2^-11 relative plus f32 product noise
    assert (np.abs(w - want) <= np.abs(want) * 6e-4 + 1e-7).all()
    assert (w[want == 0] == 0).all()  # the zeros of the lattice points stay zeros
    x = synth.make_activation(d_in, 0x99, np.float16, batch=1100 if d_out == 40 else 20)
    y = rt.forward_batch_dense(proj, torch.from_numpy(x).cuda()).cpu().numpy()
    ref = oracle.gemv_f64(m.codes, d_out, d_in, m.centroids, m.row_scales, tail16, x.astype(np.float64))
    assert rel_l2(y, ref) <= TOL_F16
    assert not rt.poll_range_error()


def test_greedy_head_kernel_matches_a_float_argmax(rt):
    """llvq_op_lm_head_argmax_h: f32 logits of an f16 embedding shard, lowest row on ties, row offset added."""
    torch = _torch()
    from llvq_b200.model import kernel_head
    head = kernel_head(rt.lib)
    g = torch.Generator(device="cuda").manual_seed(4)
    for rows, hidden in ((151936, 2560), (1000, 64), (7, 8), (18992, 5120)):
        e = (0.02 * torch.randn(rows, hidden, device="cuda", generator=g)).half()
        h = torch.randn(hidden, device="cuda", generator=g).half()
        logits = e.float() @ h.float()
        val, idx = head(e, h, 1000)
        torch.cuda.synchronize()
        assert int(idx) - 1000 == int(logits.argmax()), (rows, hidden)
        assert abs(float(val) - float(logits.max())) <= 1e-4 * max(1.0, abs(float(logits.max())))
        # a shard of the rows reports the same logit for the same row (nothing depends on the split)
        lo = rows // 3
        v2, i2 = head(e[lo:], h, lo)
        if int(logits.argmax()) >= lo:
            assert int(i2) == int(logits.argmax()) and float(v2) == float(val)
    e = torch.zeros(64, 16, device="cuda", dtype=torch.float16)
    e[5] = 1.0
    e[9] = 1.0
    _, idx = head(e, torch.ones(16, device="cuda", dtype=torch.float16), 0)
    assert int(idx) == 5
    with pytest.raises(Exception):
        head(torch.zeros(4, 12, device="cuda", dtype=torch.float16), torch.zeros(12, device="cuda", dtype=torch.float16), 0)


def _tp_regions(L, n, data_bytes):
    import ctypes as C
    from llvq_b200._lib import check
    regions = (C.c_void_p * n)()
    for r in range(n):
        p, h = C.c_void_p(), (C.c_uint8 * 64)()
        check(L.llvq_tp_region_create(0, data_bytes, C.byref(p), h))
        regions[r] = p.value
    return regions


def test_peer_exchange_protocol_with_all_ranks_in_one_cooperative_launch(rt):
    """llvq_tp_exchange on one GPU: four ranks' regions in the same memory, the four exchanges run as ONE
    cooperative launch (ranks that wait on each other are never separate launches on a GPU). Every region
    ends up with all shards in rank order, over several rounds and two sites, with aligned and odd sizes."""
    import ctypes as C
    torch = _torch()
    from llvq_b200._lib import check
    from llvq_b200.parallel import _DeviceBytes
    L, n = rt.lib, 4
    flag_bytes, buf_bytes = 512, 4096
    regions = _tp_regions(L, n, 2 * buf_bytes)
    ctxs = (C.c_void_p * n)()
    for r in range(n):
        c = C.c_void_p()
        check(L.llvq_tp_ctx_create(0, r, n, regions, 0, C.byref(c)))
        ctxs[r] = c.value
    views = [torch.as_tensor(_DeviceBytes(regions[r], flag_bytes + 2 * buf_bytes), device="cuda") for r in range(n)]
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator(device="cuda").manual_seed(1)
    for rnd, (site, shard_bytes) in enumerate([(0, 640), (1, 1001), (0, 16), (1, 2), (0, 1024)]):
        shards = [torch.randint(0, 256, (shard_bytes,), dtype=torch.uint8, device="cuda", generator=g) for _ in range(n)]
        srcs = (C.c_void_p * n)(*[s.data_ptr() for s in shards])
        off = flag_bytes + site * buf_bytes
        check(L.llvq_tp_exchange_emulated(ctxs, n, site, off, srcs, shard_bytes, st))
        torch.cuda.synchronize()
        want = torch.cat(shards)
        for r in range(n):
            assert torch.equal(views[r][off:off + n * shard_bytes], want), (rnd, r)
            flags = views[r][:flag_bytes].view(torch.int32).view(16, 8)
            assert flags[site, :n].tolist() == [rnd + 1] * n  # every source released exchange number rnd + 1 here
    for r in range(n):
        err = C.c_int32(-1)
        check(L.llvq_tp_poll_error(ctxs[r], C.byref(err)))
        assert err.value == 0
        L.llvq_tp_ctx_destroy(ctxs[r])
    del views
    for r in range(n):
        check(L.llvq_tp_region_free(0, regions[r]))


def test_peer_exchange_wait_runs_out_and_reports_instead_of_hanging(rt):
    """A peer that never shows up: the bounded wait gives up, the kernel returns, the error word says so and
    the rank's own shard has still been delivered (nothing is made to fault or hang)."""
    import ctypes as C
    torch = _torch()
    from llvq_b200._lib import check
    from llvq_b200.parallel import _DeviceBytes
    L = rt.lib
    regions = _tp_regions(L, 2, 1024)
    c = C.c_void_p()
    check(L.llvq_tp_ctx_create(0, 0, 2, regions, 2000, C.byref(c)))  # rank 0 of 2; rank 1 never runs
    shard = torch.arange(64, dtype=torch.uint8, device="cuda")
    check(L.llvq_tp_exchange(c, 3, 512, C.c_void_p(shard.data_ptr()), 64, C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    err = C.c_int32(0)
    check(L.llvq_tp_poll_error(c, C.byref(err)))
    assert err.value == 4
    check(L.llvq_tp_poll_error(c, C.byref(err)))
    assert err.value == 0  # reading clears it
    peer = torch.as_tensor(_DeviceBytes(regions[1], 512 + 1024), device="cuda")
    assert torch.equal(peer[512:576], shard) and int(peer[:512].view(torch.int32).view(16, 8)[3, 0]) == 1
    assert L.llvq_tp_exchange(c, 16, 512, C.c_void_p(shard.data_ptr()), 64, None) != 0   # site out of range
    assert L.llvq_tp_exchange(c, 0, 100, C.c_void_p(shard.data_ptr()), 64, None) != 0    # offset inside the flags
    L.llvq_tp_ctx_destroy(c)
    del peer
    for r in range(2):
        check(L.llvq_tp_region_free(0, regions[r]))


@pytest.mark.parametrize("d_out,d_in", [(200, 24 * 70 + 9), (64, 24 * 480 + 8), (40, 24 * 700 + 3), (24, 24 * 33),
                                        (1000, 24 * 5 + 1), (3, 24 * 300), (16, 7)])
def test_gemv_column_chunks_and_odd_shapes(rt, oracle, d_out, d_in):
    """Rows too long for one buffer of activation digits are cut into column chunks whose partial row sums are
    added in chunk order (f16 activations: beyond 472 blocks; f32: beyond 292); a handful of rows leaves most CTAs
    and one warp group idle; 7 columns are a tail-only matrix. Every shape gives the oracle's value within the
    tolerance of its activation type and the same bits on every launch."""
    torch = _torch()
    from llvq_b200 import synth
    m = synth.make_matrix(d_out, d_in, 0x6A1D + d_out)
    proj = rt.upload(m, tail_f16=True)
    tail16 = m.tail.astype(np.float16).astype(np.float32)
    for dt, tol in ((np.float16, TOL_F16), (np.float32, TOL_F32)):
        x = torch.from_numpy(synth.make_activation(d_in, 3, dt)).cuda()
        ref = oracle.gemv_f64(m.codes, d_out, d_in, m.centroids, m.row_scales, tail16, x.cpu().numpy().astype(np.float64))
        y = rt.forward(proj, x).clone()
        assert rel_l2(y.cpu().numpy(), ref) <= tol, dt
        for _ in range(3):
            assert torch.equal(rt.forward(proj, x), y)
    proj.free()
    assert not rt.poll_range_error()


@pytest.mark.parametrize("d_out,d_in", [(640, 2560), (300, 9728), (96, 17408), (64, 48), (2000, 24 * 40 + 10)])
def test_gemv_with_the_norm_or_the_swiglu_product_in_the_kernel(rt, d_out, d_in):
    """llvq_gemv_norm_h and llvq_gemv_silu_h form the projection's activation in its staging step. Both give
    the bits of the two-kernel sequence (llvq_op_add_rmsnorm_h or llvq_op_silu_mul_h, then llvq_gemv_h) and
    the norm variant leaves x + delta in the other stream buffer, with and without a delta, for rows with a tail,
    without one, and long enough to be cut into column chunks."""
    import ctypes as C
    torch = _torch()
    from llvq_b200 import synth
    from llvq_b200._lib import check
    L = rt.lib
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: C.c_void_p(t.data_ptr())
    m = synth.make_matrix(d_out, d_in, 0x5EED + d_in)
    proj = rt.upload(m, tail_f16=True)
    g = torch.Generator(device="cuda").manual_seed(d_in)
    resid = (torch.randn(d_in, device="cuda", generator=g) * 1.7).half()
    delta = (torch.randn(d_in, device="cuda", generator=g) * 0.4).half()
    w = (1.0 + 0.05 * torch.randn(d_in, device="cuda", generator=g)).half()
    eps = 1e-6
    if d_in % 2 == 0 and d_in <= 16384:  # the norm kernels' limit
        for d in (delta, None):
            x = resid.clone()
            h = torch.empty_like(x)
            check(L.llvq_op_add_rmsnorm_h(p(x), p(d) if d is not None else None, p(w), p(h), d_in, eps, st))
            want = rt.forward(proj, h).clone()
            x_out = torch.full_like(resid, float("nan"))
            got = rt.forward_norm(proj, resid, d, w, eps, x_out)
            assert torch.equal(x_out, x)
            assert torch.equal(got, want)
            assert torch.equal(rt.forward_norm(proj, resid, d, w, eps, x_out), want)
        with pytest.raises(RuntimeError):
            rt.forward_norm(proj, resid, delta, w, eps, resid)  # in place: refused
    if d_in % 8 == 0:
        gu = (torch.randn(2 * d_in, device="cuda", generator=g) * 2.0).half()
        act = torch.empty(d_in, dtype=torch.float16, device="cuda")
        check(L.llvq_op_silu_mul_h(p(gu), p(act), d_in, st))
        want = rt.forward(proj, act).clone()
        assert torch.equal(rt.forward_silu(proj, gu), want)
    else:
        with pytest.raises(RuntimeError):
            rt.forward_silu(proj, torch.zeros(2 * d_in, dtype=torch.float16, device="cuda"))
    proj.free()
    assert not rt.poll_range_error()


def test_overlapped_launches_keep_stream_order(rt):
    """Back-to-back fused GEMVs are launched with programmatic stream serialisation: the next launch's prologue
    runs while the previous launch drains. A chain in which every launch reads the previous launch's output
    (and overwrites a buffer the one before it read) gives the bits of ordinary launches, a hundred times over."""
    torch = _torch()
    from llvq_b200 import synth
    dims = [(2560, 4096), (4096, 2560), (2560, 4096), (1024, 2560)]
    projs = [rt.upload(synth.make_matrix(do, di, 0xD0 + i), tail_f16=True) for i, (do, di) in enumerate(dims)]
    x0 = torch.from_numpy(synth.make_activation(4096, 5, np.float16)).cuda()

    def chain():
        bufs = [x0, torch.empty(2560, dtype=torch.float16, device="cuda"), torch.empty(4096, dtype=torch.float16, device="cuda")]
        a = rt.forward(projs[0], bufs[0], out=bufs[1])
        b = rt.forward(projs[1], a, out=bufs[2])
        b.mul_(0.01)  # an ordinary kernel between two launches
        c = rt.forward(projs[2], b, out=bufs[1])   # overwrites what the second launch read
        c.mul_(0.01)
        return rt.forward(projs[3], c).clone()

    try:
        rt.set_overlap(False)
        want = chain()
        torch.cuda.synchronize()
        rt.set_overlap(True)
        for _ in range(100):
            assert torch.equal(chain(), want)
        # without the ordinary kernels in between: launch directly behind launch
        ys = [torch.empty(1024, dtype=torch.float16, device="cuda") for _ in range(50)]
        xin = torch.from_numpy(synth.make_activation(2560, 6, np.float16)).cuda()
        rt.set_overlap(False)
        ref = rt.forward(projs[3], xin).clone()
        rt.set_overlap(True)
        for y in ys:
            rt.forward(projs[3], xin, out=y)
        torch.cuda.synchronize()
        assert all(torch.equal(y, ref) for y in ys)
    finally:
        rt.set_overlap(True)
        for p in projs:
            p.free()
    assert not rt.poll_range_error()


def test_two_runtimes_on_two_devices_in_one_process(oracle):
    """The opt-in shared-memory size of a kernel is a per-device setting: a second runtime on another GPU of the
    same process must raise it again (and every launch must run on its runtime's device, whatever device is
    current). One GEMV, one batched GEMM, one rotation and one attention-free decode-step kernel on each."""
    torch = _torch()
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from llvq_b200 import FusedRuntime, synth
    m = synth.make_matrix(300, 2560, 0x2D0)  # 106 blocks + 16 tail columns; 2560 = 512 * 5 has a servable rotation
    x = synth.make_activation(m.d_in, 9, np.float16)
    tail16 = m.tail.astype(np.float16).astype(np.float32)
    ref = oracle.gemv_f64(m.codes, m.d_out, m.d_in, m.centroids, m.row_scales, tail16, x.astype(np.float64))
    outs = []
    rts = [FusedRuntime(0), FusedRuntime(1)]
    try:
        for dev, r in enumerate(rts):
            with torch.cuda.device(1 - dev):  # the "wrong" current device on purpose
                proj = r.upload(m, tail_f16=True)
                xd = torch.from_numpy(x).to(f"cuda:{dev}")
                with torch.cuda.device(dev):
                    y = r.forward(proj, xd)
                    yb = r.forward_batch(proj, xd[None, :].repeat(16, 1).contiguous())
                    rot = r.rotation(m.d_in, 77)
                    xr = r.rotate(rot, xd)
                    torch.cuda.synchronize()
                assert rel_l2(y.cpu().numpy(), ref) <= TOL_F16
                assert rel_l2(yb[3].cpu().numpy(), ref) <= TOL_F16
                outs.append((y.cpu(), xr.cpu()))
                rot.free()
                proj.free()
                assert not r.poll_range_error()
        assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    finally:
        for r in rts:
            r.close()
