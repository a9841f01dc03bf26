"""The allocation-free Dense chain (`a4c_mlp_i8_static`).

Some embedders of this library run a model from code that may not call cudaMalloc -- a callback inside another
runtime's stream, a process whose device memory belongs to its own pool, a loop that must never wait on the CUDA
allocator's lock.  For them the chain's scratch is a fixed array inside the library image.  This test calls that
entry point through the C ABI twice in a row and checks both results, bit for bit, against the ordinary
`a4c_mlp_i8` (whose scratch is allocated) and against the CPU oracle; it checks that the device's free memory
does not move across calls, that chains which take the other kernel branches (a first layer too short for the
tensor-core kernel, unsigned input and output, a single layer) agree with the oracle too, and that a problem
larger than the fixed array is refused.

The file name sorts last on purpose: a run that stops at the first failure has then already run everything else.
"""

import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _call(fn_name, x_d, lda, n, dims, wt_ptrs, ldw, b_ptrs, shifts, relus, y_d, ldy, M, status=None):
    import gpu_util as G
    from aie4ml_b200 import lib as a4c

    L = a4c.load()
    args = [x_d.data_ptr(), lda, 0, n, ctypes.cast(dims, ctypes.c_void_p), ctypes.cast(wt_ptrs, ctypes.c_void_p),
            ctypes.cast(ldw, ctypes.c_void_p), ctypes.cast(b_ptrs, ctypes.c_void_p), ctypes.cast(shifts, ctypes.c_void_p),
            ctypes.cast(relus, ctypes.c_void_p), 2, y_d.data_ptr(), ldy, 0, M]
    if fn_name == 'a4c_mlp_i8_static':
        args.append(status)
    args.append(G.stream())
    return getattr(L, fn_name)(*args)


def test_static_chain_matches_allocating_chain_twice_in_a_row():
    import torch

    import gpu_util as G

    rng = np.random.default_rng(2024)
    for dims_t, M in (((16, 64, 32, 32, 5), 1024), ((512, 1024, 1024, 16), 2048)):
        n = len(dims_t) - 1
        x = rng.integers(-128, 128, (M, dims_t[0])).astype(np.int8)
        ws = [rng.integers(-127, 128, (dims_t[i], dims_t[i + 1])).astype(np.int8) for i in range(n)]
        bs = [rng.integers(-(1 << 12), 1 << 12, dims_t[i + 1]).astype(np.int32) for i in range(n)]
        wts = [G.dev(G.pack_wt(w)) for w in ws]
        b_d = [G.dev(b) for b in bs]
        dims = (ctypes.c_int * (n + 1))(*dims_t)
        wt_ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in wts])
        ldw = (ctypes.c_int64 * n)(*[t.shape[1] for t in wts])
        b_ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in b_d])
        shifts = (ctypes.c_int * n)(*([7] * n if dims_t[0] == 16 else [9] * n))
        relus = (ctypes.c_int * n)(*([1] * (n - 1) + [0]))
        lda = (dims_t[0] + 15) // 16 * 16
        x_d = G.dev(G.padded(x, lda))
        N = dims_t[-1]
        ldy = (N + 15) // 16 * 16
        want_d = torch.zeros((M, ldy), dtype=torch.int8, device='cuda')
        assert _call('a4c_mlp_i8', x_d, lda, n, dims, wt_ptrs, ldw, b_ptrs, shifts, relus, want_d, ldy, M) == 0
        torch.cuda.synchronize()
        want = want_d.cpu().numpy()[:, :N]
        assert np.abs(want).max() > 0
        for attempt in range(2):   # the second call finds the first call's activations in the shared array
            got_d = torch.full((M, ldy), 0x5A, dtype=torch.int8, device='cuda')
            status = ctypes.c_int(-1)
            rc = _call('a4c_mlp_i8_static', x_d, lda, n, dims, wt_ptrs, ldw, b_ptrs, shifts, relus, got_d, ldy, M,
                       ctypes.byref(status))
            assert rc == 0 and status.value == 0, (attempt, rc, status.value)
            np.testing.assert_array_equal(got_d.cpu().numpy()[:, :N], want, err_msg=f'call {attempt}')
        # asynchronous form (no status read-back) gives the same bytes
        got_d = torch.zeros((M, ldy), dtype=torch.int8, device='cuda')
        assert _call('a4c_mlp_i8_static', x_d, lda, n, dims, wt_ptrs, ldw, b_ptrs, shifts, relus, got_d, ldy, M, None) == 0
        torch.cuda.synchronize()
        np.testing.assert_array_equal(got_d.cpu().numpy()[:, :N], want)


def test_static_chain_refuses_what_does_not_fit():
    import torch

    import gpu_util as G
    from aie4ml_b200 import lib as a4c

    # 8192 rows x 1024 hidden bytes = 8 MiB > the 4 MiB buffer: refused before anything is launched
    M, dims_t = 8192, (64, 1024, 16)
    n = 2
    wts = [torch.zeros((dims_t[i + 1], dims_t[i]), dtype=torch.int8, device='cuda') for i in range(n)]
    dims = (ctypes.c_int * 3)(*dims_t)
    wt_ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in wts])
    ldw = (ctypes.c_int64 * n)(64, 1024)
    b_ptrs = (ctypes.c_void_p * n)(None, None)
    shifts = (ctypes.c_int * n)(7, 7)
    relus = (ctypes.c_int * n)(1, 0)
    x_d = torch.zeros((M, 64), dtype=torch.int8, device='cuda')
    y_d = torch.full((M, 16), 0x5A, dtype=torch.int8, device='cuda')
    rc = _call('a4c_mlp_i8_static', x_d, 64, n, dims, wt_ptrs, ldw, b_ptrs, shifts, relus, y_d, 16, M, None)
    assert rc == a4c.A4C_ERR_TOO_LARGE
    assert a4c.load().a4c_error_string(rc).decode() == 'problem exceeds a stated maximum'
    torch.cuda.synchronize()
    assert (y_d.cpu().numpy() == 0x5A).all()          # nothing ran
    # exactly at the limit is accepted: 4096 rows x 1024 bytes = 4 MiB
    y2 = torch.zeros((4096, 16), dtype=torch.int8, device='cuda')
    assert _call('a4c_mlp_i8_static', x_d, 64, n, dims, wt_ptrs, ldw, b_ptrs, shifts, relus, y2, 16, 4096, None) == 0
    torch.cuda.synchronize()


def _oracle_chain(x, layers, tok, out_dtype):
    from oracle import oracle

    cur = x
    for i, (w, b, shift, relu) in enumerate(layers):
        last = i == len(layers) - 1
        cur = oracle.dense(cur, w, b, shift=shift, tok=tok, relu=relu, out_dtype=out_dtype if last else 'int8')
    return cur


def _layers(rng, dims, shift, bias=True):
    n = len(dims) - 1
    return [(rng.integers(-127, 128, (dims[i], dims[i + 1])).astype(np.int8),
             rng.integers(-(1 << 12), 1 << 12, dims[i + 1]).astype(np.int32) if bias else None, shift, i < n - 1)
            for i in range(n)]


def test_static_chain_against_the_oracle_on_every_kernel_branch_without_allocating():
    import torch

    import gpu_util as G

    rng = np.random.default_rng(77)
    cases = [
        # (dims, rows, input type, output type, rounding token)
        ((16, 64, 32, 32, 5), 1024, np.int8, 'int8', 'positive_inf'),    # tensor-core kernel in every layer
        ((8, 48, 10), 300, np.int8, 'int8', 'conv_even'),                # K = 8 < 16: the dp4a kernel takes layer 0
        ((32, 64, 24), 257, np.uint8, 'uint8', 'symmetric_inf'),         # unsigned input and output
        ((64, 40), 129, np.int8, 'int8', 'floor'),                       # a single layer: no scratch is touched
    ]
    # one warm-up call sets the array up on this device; after it the free memory must not move
    d0, r0 = cases[0][0], cases[0][1]
    G.mlp_chain(rng.integers(-128, 128, (r0, d0[0])).astype(np.int8), _layers(rng, d0, 7), tok='positive_inf',
                fn_name='a4c_mlp_i8_static')
    prepared = []
    for dims, rows, in_t, out_t, tok in cases:
        lo, hi = (0, 256) if in_t is np.uint8 else (-128, 128)
        prepared.append((rng.integers(lo, hi, (rows, dims[0])).astype(in_t), _layers(rng, dims, 7), tok, out_t))
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    for x, layers, tok, out_t in prepared:
        want = _oracle_chain(x, layers, tok, out_t)
        for attempt in range(2):
            got = G.mlp_chain(x, layers, tok=tok, out_dtype=out_t, fn_name='a4c_mlp_i8_static')
            np.testing.assert_array_equal(got.astype(np.int64), want.astype(np.int64),
                                          err_msg=f'dims {[w.shape for w, *_ in layers]} call {attempt}')
    # the calls themselves: same buffers, several sizes, free device memory read before and after
    import ctypes

    x, layers, tok, out_t = prepared[0]
    n = len(layers)
    wts = [G.dev(G.pack_wt(w)) for w, *_ in layers]
    b_d = [G.dev(b) for _, b, _, _ in layers]
    dims = (ctypes.c_int * (n + 1))(x.shape[1], *[w.shape[1] for w, *_ in layers])
    wt_ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in wts])
    ldw = (ctypes.c_int64 * n)(*[t.shape[1] for t in wts])
    b_ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in b_d])
    shifts = (ctypes.c_int * n)(*([7] * n))
    relus = (ctypes.c_int * n)(*([1] * (n - 1) + [0]))
    x_d = G.dev(x)
    y_d = torch.zeros((x.shape[0], 16), dtype=torch.int8, device='cuda')
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for rows in (1024, 1, 517, 1024):
        assert _call('a4c_mlp_i8_static', x_d, 16, n, dims, wt_ptrs, ldw, b_ptrs, shifts, relus, y_d, 16, rows, None) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, 'the allocation-free entry point changed the free device memory'
