"""The allocation-free decode-attention entry point, called the way its intended users call it:
through the exported C symbol of libgvirt_kernels.so with raw pointers, without this package's
Python op layer and without handing it any scratch buffer.

Those users are callers that may not allocate device memory (a plug-in living inside another
framework's memory pool, code inside a no-allocation region such as a fixed-budget serving loop, a
plain C host program). The check: two calls in a row (different inputs, the second one re-using
the library's built-in scratch with the first call's leftovers in it) must both match the regular
entry point, which gets explicit scratch from the caller. The file name keeps this test last in
collection order so that a run that stops at the first failure has already run everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from gvirt_b200 import build
    path = build.kernels_lib_path()
    if not path.exists():
        build.build_kernels()
    lib = ctypes.CDLL(str(path))
    lib.gv_last_error.restype = ctypes.c_char_p
    return lib


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _case(seed, batch, nq, nkv, hd, bs, lens):
    g = torch.Generator().manual_seed(seed)
    nblk_per = [(l + bs - 1) // bs for l in lens]
    num_blocks = sum(nblk_per) + 2
    perm = torch.randperm(num_blocks, generator=g).tolist()
    bt = torch.zeros(batch, max(nblk_per) + 1, dtype=torch.int32)
    k = 0
    for b in range(batch):
        for j in range(nblk_per[b]):
            bt[b, j] = perm[k]
            k += 1
    kc = (torch.randn(num_blocks, bs, nkv, hd, generator=g) * 0.5).bfloat16().cuda()
    vc = (torch.randn(num_blocks, bs, nkv, hd, generator=g) * 0.5).bfloat16().cuda()
    q = (torch.randn(batch, nq * hd, generator=g) * 0.3).bfloat16().cuda()
    return q, kc, vc, bt.cuda(), torch.tensor(lens, dtype=torch.int32).cuda(), num_blocks


def _regular(lib, q, kc, vc, bt, lens, nq, nkv, hd, bs, nsplit, num_blocks):
    batch = q.shape[0]
    out = torch.empty_like(q)
    po = torch.empty(batch * nq * nsplit * hd, dtype=torch.float32, device="cuda")
    pl = torch.empty(batch * nq * nsplit, dtype=torch.float32, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ll = ctypes.c_longlong
    rc = lib.gv_paged_attention_decode(_p(q), _p(kc), _p(vc), _p(bt), _p(lens), _p(out), _p(po), _p(pl),
                                       ll(batch), ll(nq), ll(nkv), ll(hd), ll(bs), ll(bt.shape[1]),
                                       ll(nsplit), ctypes.c_float(1.0), ll(num_blocks), stream)
    assert rc == 0, lib.gv_last_error()
    return out


def _noalloc(lib, q, kc, vc, bt, lens, nq, nkv, hd, bs, nsplit, num_blocks):
    batch = q.shape[0]
    out = torch.empty_like(q)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ll = ctypes.c_longlong
    rc = lib.gv_paged_attention_decode_noalloc(_p(q), _p(kc), _p(vc), _p(bt), _p(lens), _p(out),
                                               ll(batch), ll(nq), ll(nkv), ll(hd), ll(bs),
                                               ll(bt.shape[1]), ll(nsplit), ctypes.c_float(1.0),
                                               ll(num_blocks), stream)
    return rc, out


def test_noalloc_matches_regular_entry_point_twice():
    lib = _lib()
    nq, nkv, hd, bs = 16, 4, 128, 128
    for call, (seed, lens, nsplit) in enumerate([(11, [300, 1, 1025, 77, 640], 3), (12, [90, 2048, 5, 129, 400], 4)]):
        q, kc, vc, bt, sl, nb = _case(seed, len(lens), nq, nkv, hd, bs, lens)
        want = _regular(lib, q, kc, vc, bt, sl, nq, nkv, hd, bs, nsplit, nb)
        rc, got = _noalloc(lib, q, kc, vc, bt, sl, nq, nkv, hd, bs, nsplit, nb)
        assert rc == 0, lib.gv_last_error()
        torch.cuda.synchronize()
        err = (got.float() - want.float()).abs().max().item()
        assert torch.isfinite(got.float()).all()
        assert err <= 1e-2, f"call {call}: max |noalloc - regular| = {err}"
    st = ctypes.c_uint(0)
    assert lib.gv_noalloc_status_read(ctypes.byref(st), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    assert st.value == 0


def test_noalloc_rejects_oversized_request():
    lib = _lib()
    nq, nkv, hd, bs = 32, 8, 128, 128
    lens = [64] * 64
    q, kc, vc, bt, sl, nb = _case(13, len(lens), nq, nkv, hd, bs, lens)
    rc, _ = _noalloc(lib, q, kc, vc, bt, sl, nq, nkv, hd, bs, 16, nb)  # 64*32*16*129*4 B > 8 MiB
    assert rc == -4
    assert b"exceeds" in lib.gv_last_error()


def test_noalloc_flags_a_length_beyond_the_block_table_and_the_flag_can_be_cleared():
    """Raw callers bypass the host-side metadata checks, so the kernel itself must refuse a
    sequence length that runs past the block-table row: the keys beyond the row are skipped (no
    read outside the table), GV_ST_BAD_INDEX (32) is raised, and `gv_noalloc_status_reset` clears
    the sticky word so that the next, valid call reads 0 again."""
    lib = _lib()
    nq, nkv, hd, bs = 8, 2, 128, 128
    lens = [200, 260]
    q, kc, vc, bt, sl, nb = _case(14, len(lens), nq, nkv, hd, bs, lens)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    st = ctypes.c_uint(0)
    bad = sl.clone()
    bad[1] = bt.shape[1] * bs + 40          # 40 keys past the end of the row
    rc, got = _noalloc(lib, q, kc, vc, bt, bad, nq, nkv, hd, bs, 2, nb)
    assert rc == 0, lib.gv_last_error()
    assert lib.gv_noalloc_status_read(ctypes.byref(st), stream) == 0
    assert st.value & 32
    assert torch.isfinite(got.float()).all()
    assert lib.gv_noalloc_status_reset(stream) == 0
    want = _regular(lib, q, kc, vc, bt, sl, nq, nkv, hd, bs, 2, nb)
    rc, got = _noalloc(lib, q, kc, vc, bt, sl, nq, nkv, hd, bs, 2, nb)
    assert rc == 0, lib.gv_last_error()
    assert lib.gv_noalloc_status_read(ctypes.byref(st), stream) == 0
    assert st.value == 0
    assert (got.float() - want.float()).abs().max().item() <= 1e-2
