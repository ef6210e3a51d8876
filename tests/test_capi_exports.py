"""The C-ABI library builds, loads and exports every symbol include/b200tp.h declares.
No compute call is made (no GPU needed)."""
import ctypes
import re
from pathlib import Path

import pytest

from mlx_train_perf_b200 import _lib
from mlx_train_perf_b200.build import build

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    build(verbose=False)
    return _lib.load()


def _declared_symbols():
    text = (ROOT / "include" / "b200tp.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200tp_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = _declared_symbols()
    assert len(names) >= 11
    raw = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in names:
        assert hasattr(raw, name), f"{name} declared in include/b200tp.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes signatures out of sync with the header"


def test_status_strings_and_version(lib):
    assert lib.b200tp_version() >= 100
    assert lib.b200tp_status_string(0) == b"ok"
    for code in (1, 2, 3, 4, 5, 6, 7, 101, 102, 103, 104):
        assert lib.b200tp_status_string(code) not in (b"", b"unknown status")
    assert lib.b200tp_status_string(9999) == b"unknown status"


def test_host_side_refusals_need_no_gpu(lib):
    a = _lib.CeArgs()
    a.n, a.d, a.v_local = 0, 64, 128
    assert lib.b200tp_linear_ce_fwd_workspace_bytes(ctypes.byref(a)) == 0
    assert b"at least one row" in lib.b200tp_last_error()
    b = _lib.AttnArgs()
    b.b, b.hq, b.hkv, b.s, b.d, b.dtype, b.causal = 1, 6, 4, 128, 128, _lib.BF16, 1
    assert lib.b200tp_flash_bwd_workspace_bytes(ctypes.byref(b)) == 0
    assert b"multiple of Hkv" in lib.b200tp_last_error()
    b.hq, b.d = 8, 80
    assert lib.b200tp_flash_bwd_workspace_bytes(ctypes.byref(b)) == 0
    assert b"head_dim" in lib.b200tp_last_error()


def test_workspace_sizes_hold_no_full_logits(lib):
    """The zero-(N,V) claim is auditable from the workspace sizes: at the flagship shape the
    forward needs a few MB of partial triples, the backward one (N, 15360) bf16 chunk of g (a tenth of the
    vocabulary) + an fp32 (N, D) accumulator -- far below the 2.5 GB a bf16 (N, V) tensor would take."""
    a = _lib.CeArgs()
    a.hidden = a.weight = a.targets = 1 << 20   # non-null placeholders; nothing is dereferenced
    a.n, a.d, a.v_local, a.dtype, a.impl = 8192, 4096, 151936, _lib.BF16, 0
    fwd = lib.b200tp_linear_ce_fwd_workspace_bytes(ctypes.byref(a))
    bwd = lib.b200tp_linear_ce_bwd_workspace_bytes(ctypes.byref(a), _lib.BF16)
    assert 0 < fwd < 64 << 20
    assert 0 < bwd <= 8192 * 15360 * 2 + 8192 * 4096 * 4 + 4096      # ten balanced chunks of 15360 vocab rows
    assert bwd < 8192 * 151936 * 2 // 4
    a.n = 65536                                   # large N: the bound drops so that the g tile stays within 512 MiB
    assert lib.b200tp_linear_ce_bwd_workspace_bytes(ctypes.byref(a), _lib.BF16) <= (512 << 20) + 65536 * 4096 * 4 + 4096
    a.n = 8192
    # the chunk bound is the caller's to lower: 16 x 256 = 4096 vocab rows per chunk -> a quarter of the scratch for g
    a.reserved = 16
    small = lib.b200tp_linear_ce_bwd_workspace_bytes(ctypes.byref(a), _lib.BF16)
    assert 0 < small <= 8192 * 4096 * 2 + 8192 * 4096 * 4 + 4096
    # a 4-bit head expanded inside the kernels (0x10000) adds no dequantised chunk to either workspace; the
    # chunked form (the default at this row count) adds one bf16 chunk of the head
    a.weight, a.w_q, a.scales, a.biases = None, 1 << 20, 1 << 20, 1 << 20
    a.quant_bits, a.group_size, a.qparam_dtype = 4, 64, _lib.BF16
    bwd_q = bwd
    a.reserved = 0x10000
    assert lib.b200tp_linear_ce_fwd_workspace_bytes(ctypes.byref(a)) == fwd
    assert bwd_q <= lib.b200tp_linear_ce_bwd_workspace_bytes(ctypes.byref(a), _lib.BF16) <= bwd_q + 1024
    a.reserved = 0
    chunk = 15360 * 4096 * 2                      # ceil(151936 / 10) vocab rows, padded to a multiple of 256
    assert lib.b200tp_linear_ce_fwd_workspace_bytes(ctypes.byref(a)) >= fwd + chunk - 4096
    assert bwd_q + chunk <= lib.b200tp_linear_ce_bwd_workspace_bytes(ctypes.byref(a), _lib.BF16) <= bwd_q + chunk + 1024
    a.n = 512                                     # few rows: the forward expands in the kernel by default,
    assert lib.b200tp_linear_ce_fwd_workspace_bytes(ctypes.byref(a)) < 1 << 20
    bwd512 = lib.b200tp_linear_ce_bwd_workspace_bytes(ctypes.byref(a), _lib.BF16)
    assert bwd512 >= chunk                         # the backward stays chunked (one bf16 chunk of the head) ...
    a.reserved = 0x10000
    assert lib.b200tp_linear_ce_bwd_workspace_bytes(ctypes.byref(a), _lib.BF16) == bwd512 - chunk   # ... unless forced
    a.reserved = 0x30000
    assert lib.b200tp_linear_ce_fwd_workspace_bytes(ctypes.byref(a)) == 0 and b"selectors" in lib.b200tp_last_error()


def _attn_shape(hq, hkv, s, b=1, reserved=0):
    a = _lib.AttnArgs()
    a.b, a.hq, a.hkv, a.s, a.d, a.dtype, a.causal, a.scale = b, hq, hkv, s, 128, _lib.BF16, 1, 128 ** -0.5
    for arr, h in ((a.q_stride, hq), (a.k_stride, hkv), (a.v_stride, hkv), (a.o_stride, hq)):
        arr[0], arr[1], arr[2] = h * s * 128, s * 128, 128
    a.impl, a.reserved = 0, reserved
    return a


def test_attention_workspace_sizes_are_linear_in_s(lib):
    """Attention scratch is O(S): at the flagship shape (a grid that fills the SMs) the forward needs
    none and the backward the row statistics as a bf16 operand tile of 32 bytes per row (dK / dV CTAs walk
    whole GQA groups: no partials); one
    kv-head group of the same sequence (the 8-GPU share) gets the split forward's fp32 partials and the
    per-q-head dK / dV partials -- still nothing like an (S, S) matrix (256 MiB per head in fp32)."""
    vec = 32 * 8192 * 4
    big = _attn_shape(32, 8, 8192)
    assert lib.b200tp_flash_fwd_workspace_bytes(ctypes.byref(big)) == 0
    assert lib.b200tp_flash_bwd_workspace_bytes(ctypes.byref(big)) <= 8 * vec + 1024
    per_head = _attn_shape(32, 8, 8192, reserved=64)           # forced per-q-head CTAs: the partials come back
    assert lib.b200tp_flash_bwd_workspace_bytes(ctypes.byref(per_head)) >= 2 * 32 * 8192 * 128 * 4
    share = _attn_shape(4, 1, 8192)
    fwd = lib.b200tp_flash_fwd_workspace_bytes(ctypes.byref(share))
    assert 2 * 4 * 8192 * 130 * 4 <= fwd <= 4 * 4 * 8192 * 130 * 4 + 4096
    bwd = lib.b200tp_flash_bwd_workspace_bytes(ctypes.byref(share))
    assert 2 * 4 * 8192 * 128 * 4 <= bwd <= 2 * 4 * 8192 * 128 * 4 + 8 * 4 * 8192 * 4 + 4096
    assert max(fwd, bwd) < 8192 * 8192 * 4 // 4
    mha = _attn_shape(8, 8, 8192)                               # no GQA: never any partials; odd group: no split
    assert lib.b200tp_flash_bwd_workspace_bytes(ctypes.byref(mha)) <= 8 * 8 * 8192 * 4 + 1024
    assert lib.b200tp_flash_fwd_workspace_bytes(ctypes.byref(mha)) == 0
