"""CPU: the C-ABI library loads, exports every symbol the header declares,
validates its arguments on the host and refuses to compute without a GPU."""
import ctypes as C
import os
import re
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, 'include', 'bsx.h')).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(bsx_[a-z0-9_]+)\s*\(', text)))


def test_every_declared_symbol_is_exported_and_bound(bsx):
    from brainstate_b200 import _lib
    names = header_symbols()
    assert len(names) >= 20
    for name in names:
        assert hasattr(bsx, name), f'{name} declared in include/bsx.h but not exported'
        assert name in _lib.SIGNATURES, f'{name} has no ctypes signature'
    assert set(_lib.SIGNATURES) - set(_lib.INTERNAL) <= set(names)
    assert not set(_lib.INTERNAL) & set(names), 'tuning hooks do not belong in the public header'
    assert bsx.bsx_version() == 100


def test_struct_layout_matches_header(bsx):
    from brainstate_b200._lib import BsxConn
    assert C.sizeof(BsxConn) == 4 * 8 + 8 + 8 + 4 + 4 + 8
    assert BsxConn.weights.offset == 56


@pytest.mark.parametrize('n_post', [1, 2, 40, 4000, 65536, 100003])
def test_host_generator_bit_exact_to_numpy(bsx, n_post):
    from brainstate_b200.nn import fixed_num_indices
    for seed in (0, 123, 4242):
        ref = np.random.RandomState(seed).randint(0, n_post, size=(29, 13)).astype(np.int32)
        assert np.array_equal(fixed_num_indices(seed, 29, n_post, 13), ref)


def test_host_generator_row_and_column_windows(bsx):
    seed, n_pre, n_post, K = 99, 50, 1000, 20
    full = np.random.RandomState(seed).randint(0, n_post, size=(n_pre, K)).astype(np.int32)
    # a row window replays the stream and keeps only its rows
    out = np.empty((10, K), np.int32)
    n = bsx.bsx_host_fixed_num_indices(seed, n_pre, n_post, K, 20, 30, 0, 0, out.ctypes.data, None)
    assert n == out.size and np.array_equal(out, full[20:30])
    # a column window yields the CSR block of one postsynaptic shard
    c0, c1 = 250, 500
    buf = np.empty(n_pre * K, np.int32)
    counts = np.empty(n_pre, np.int32)
    n = bsx.bsx_host_fixed_num_indices(seed, n_pre, n_post, K, 0, n_pre, c0, c1, buf.ctypes.data, counts.ctypes.data)
    keep = (full >= c0) & (full < c1)
    assert n == keep.sum()
    assert np.array_equal(counts, keep.sum(axis=1))
    assert np.array_equal(buf[:n], (full[keep] - c0))
    # bad ranges are refused with a message
    assert bsx.bsx_host_fixed_num_indices(seed, n_pre, n_post, K, 30, 20, 0, 0, out.ctypes.data, None) == -1
    assert b'row range' in bsx.bsx_last_error_string()


def test_argument_validation_needs_no_gpu(bsx):
    from brainstate_b200._lib import BsxConn, BSX_ERR_INVALID_ARG
    st = BsxConn()
    st.n_pre, st.n_post, st.conn_num, st.nnz = 4, 4, 2, 8
    assert bsx.bsx_event_vecmat(None, None, 0, 1, None, 0, None, 0, None) == BSX_ERR_INVALID_ARG
    assert bsx.bsx_event_vecmat(C.byref(st), None, 0, 1, None, 0, None, 0, None) == BSX_ERR_INVALID_ARG
    assert b'indices' in bsx.bsx_last_error_string()
    st.nnz = 7
    dummy = (C.c_float * 8)()
    st.indices = C.addressof(dummy)
    st.weights = C.addressof(dummy)
    assert bsx.bsx_float_matvec(C.byref(st), None, 1, None, None) == BSX_ERR_INVALID_ARG
    assert b'nnz' in bsx.bsx_last_error_string()
    assert bsx.bsx_status_name(-3) == b'BSX_ERR_INDEX_RANGE'
    assert bsx.bsx_event_vecmat_workspace_bytes(2, 100) >= 16 + 800
    assert bsx.bsx_transpose_workspace_bytes(10, 10, 50) >= 4 * 11 + 4 * 50
    # sliced layout: one slice per 32 768 columns; its entry points validate on the host too
    assert [bsx.bsx_sliced_slices(n) for n in (0, 1, 32768, 32769, 65536, 131072, 131073)] == [0, 1, 1, 2, 2, 4, 5]
    st.nnz = 8
    assert bsx.bsx_sliced_build(C.byref(st), None, None, None, None) == BSX_ERR_INVALID_ARG
    assert b's_indptr' in bsx.bsx_last_error_string()
    assert bsx.bsx_event_vecmat_sliced(C.byref(st), None, 0, 1, None, 0, None) == BSX_ERR_INVALID_ARG
    assert b'64-bit' in bsx.bsx_last_error_string()
    assert bsx.bsx_event_vecmat_variant(C.byref(st), 9, 4) == BSX_ERR_INVALID_ARG
    assert bsx.bsx_event_vecmat_variant(C.byref(st), 0, 4) in (0, 1)
    # compressed form of the sliced layout
    assert bsx.bsx_event_vecmat_sliced16(C.byref(st), None, None, None, 0, 1, None, 0, 0, None) == BSX_ERR_INVALID_ARG
    assert b'64-bit' in bsx.bsx_last_error_string()
    assert bsx.bsx_event_vecmat_sliced16(C.byref(st), None, None, None, 0, 1, None, 0, 31, None) == BSX_ERR_INVALID_ARG
    assert bsx.bsx_quantize_f32(None, 8, 3, None, None) == BSX_ERR_INVALID_ARG
    assert b'NULL' in bsx.bsx_last_error_string()
    assert bsx.bsx_quantize_f32(None, 0, 3, None, None) == 0             # nothing to do
    assert bsx.bsx_quantize_f32(C.addressof(dummy), 8, 40, C.addressof(dummy), None) == BSX_ERR_INVALID_ARG
    assert b'scale_log2' in bsx.bsx_last_error_string()


def test_no_cpu_fallback(bsx):
    """Without a GPU the compute entry points fail loudly; they never compute on the host."""
    import torch
    if torch.cuda.is_available():
        pytest.skip('a CUDA device is present')
    from brainstate_b200._lib import BsxConn, BSX_ERR_CUDA
    assert bsx.bsx_device_count() == 0
    idx = np.zeros(8, np.int32); w = np.ones(8, np.float32)
    spk = np.ones(4, np.uint8); out = np.full(4, 7.0, np.float32)
    ws = np.zeros(1024, np.uint8)
    st = BsxConn()
    st.n_pre, st.n_post, st.conn_num, st.nnz = 4, 4, 2, 8
    st.indices, st.weights, st.hetero = idx.ctypes.data, w.ctypes.data, 1
    rc = bsx.bsx_event_vecmat(C.byref(st), spk.ctypes.data, 0, 1, out.ctypes.data, 0, ws.ctypes.data, ws.size, None)
    assert rc == BSX_ERR_CUDA
    assert np.all(out == 7.0)
    from brainstate_b200.nn import EventFixedProb
    with pytest.raises(RuntimeError, match='GPU only'):
        EventFixedProb(20, 40, 0.1, 1.0, seed=1)


def test_layer_validation_errors_match_the_reference(bsx):
    from brainstate_b200.nn import FixedNumConn, EventFixedProb, EventFixedNumConn, init_indices_without_replace
    assert EventFixedProb is EventFixedNumConn
    with pytest.raises(AssertionError):
        FixedNumConn(20, 40, 0.1, 1.0, efferent_target='sideways', seed=1)
    with pytest.raises(AssertionError):
        FixedNumConn(20, 40, 0.1, 1.0, afferent_ratio=1.5, seed=1)
    with pytest.raises(AssertionError):
        FixedNumConn(20, 40, 1.5, 1.0, seed=1)
    for kw in ({}, {'afferent_ratio': 0.5}):
        with pytest.raises(NotImplementedError):
            FixedNumConn(20, 40, 0.2, 1.0, efferent_target='pre', seed=1, **kw)
    with pytest.raises(ValueError, match='Unknown method'):
        init_indices_without_replace(3, 5, 10, seed=1, method='bogus')
    idx = init_indices_without_replace(4, 6, 10, seed=7, method='for_loop')
    assert idx.shape == (6, 4) and idx.min() >= 0 and idx.max() < 10
    assert all(len(set(r.tolist())) == 4 for r in idx)
    assert np.array_equal(idx, init_indices_without_replace(4, 6, 10, seed=7, method='vmap'))


def test_product_path_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, 'brainstate_b200')
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith(('.py', '.cu', '.cuh', '.h')):
                text = open(os.path.join(dirpath, f)).read()
                assert 'oracle' not in text.replace('c_oracle', 'oracle') or f == 'never', (dirpath, f)


def test_shard_kernel_entry_point_validates_on_the_host(bsx):
    """bsx_net_run_sharded rejects inconsistent descriptions before anything is launched
    (no device is needed for these paths)."""
    from brainstate_b200._lib import BsxNetShard, BsxNetLinks, BsxLifParams, BSX_ERR_INVALID_ARG
    net, links, par = BsxNetShard(), BsxNetLinks(), BsxLifParams()
    call = lambda: bsx.bsx_net_run_sharded(C.byref(net), C.byref(par), C.byref(links), 10, 0, None, None, None)
    assert bsx.bsx_net_run_sharded(None, C.byref(par), C.byref(links), 1, 0, None, None, None) == BSX_ERR_INVALID_ARG
    assert call() == BSX_ERR_INVALID_ARG and b'sizes' in bsx.bsx_last_error_string()
    net.n_global, net.n_exc, net.first, net.n_local = 640, 512, 0, 640
    net.exc.n_pre, net.exc.n_post, net.inh.n_pre, net.inh.n_post = 512, 640, 128, 640
    buf = (C.c_float * 4)()
    for f in ('V', 'g_e', 'g_i', 'ref', 'incr_e', 'incr_i'):
        setattr(net, f, C.addressof(buf))
    net.ring, net.delay_e, net.delay_i = 2, 3, 1
    assert call() == BSX_ERR_INVALID_ARG and b'increment ring' in bsx.bsx_last_error_string()
    net.ring = 5
    links.world, links.rank = 17, 0
    assert call() == BSX_ERR_INVALID_ARG and b'world' in bsx.bsx_last_error_string()
    links.world, links.rank = 2, 0
    assert call() == BSX_ERR_INVALID_ARG and b'sync' in bsx.bsx_last_error_string()
    links.sync = C.addressof(buf)
    links.blocks, links.words_per_block, links.words_per_rank = 1, 8, 20
    assert call() == BSX_ERR_INVALID_ARG and b'words_per_block' in bsx.bsx_last_error_string()
    links.blocks, links.words_per_block = 1, 32
    links.slack = 2                                           # above min(delay) = 1
    assert call() == BSX_ERR_INVALID_ARG and b'slack' in bsx.bsx_last_error_string()
    links.slack, links.slots = 1, 3                           # needs 2 * slack + 2
    assert call() == BSX_ERR_INVALID_ARG and b'slots' in bsx.bsx_last_error_string()
    links.slots = 4
    assert call() == BSX_ERR_INVALID_ARG and b'inbox' in bsx.bsx_last_error_string()
    assert bsx.bsx_net_inbox_bytes(2, 3, 32, 4) == 4 * 2 * 3 * (1 + 32 * 32) * 8
    assert bsx.bsx_net_inbox_bytes(0, 3, 32, 4) == 0


def test_xla_ffi_shim_type_checks_against_a_stub_header():
    """ffi/bsx_ffi.cc compiles only where jaxlib's FFI headers exist.  Against a
    declarations-only stand-in (tests/stubs) the translation unit must parse and every
    handler's signature must match its binding (the stand-in's macro asserts it)."""
    import shutil
    import subprocess
    gxx = shutil.which('g++')
    if gxx is None:
        pytest.skip('no g++')
    cuda_inc = '/usr/local/cuda/include'
    if not os.path.exists(os.path.join(cuda_inc, 'cuda_runtime_api.h')):
        pytest.skip('no CUDA headers')
    r = subprocess.run([gxx, '-std=c++17', '-fsyntax-only', '-I', os.path.join(ROOT, 'include'),
                        '-I', os.path.join(ROOT, 'tests', 'stubs'), '-I', cuda_inc,
                        os.path.join(ROOT, 'ffi', 'bsx_ffi.cc')], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    text = open(os.path.join(ROOT, 'ffi', 'bsx_ffi.cc')).read()
    for target in ('bsx_ffi_vecmat', 'bsx_ffi_matvec', 'bsx_ffi_vecmat_vjp', 'bsx_ffi_dense_event_vecmat'):
        assert f'XLA_FFI_DEFINE_HANDLER_SYMBOL({target},' in text


def test_jax_binding_is_import_guarded():
    """The JAX registration module must not be pulled in by the package, and without jax it
    fails with a message that says what is missing."""
    import importlib
    import brainstate_b200
    assert 'brainstate_b200.jax_binding' not in sys.modules
    try:
        import jax  # noqa: F401
    except ImportError:
        with pytest.raises(ImportError, match='needs jax'):
            importlib.import_module('brainstate_b200.jax_binding')
