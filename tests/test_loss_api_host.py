"""Host-side validation of the loss / attention surfaces (no GPU): the typed refusals of
core/loss.py:126-186 and attention/api.py:52-123 of the reference."""
import pytest
import torch

from mlx_train_perf_b200.attention.api import resolve_attention_impl
from mlx_train_perf_b200.attention.segments import PackedMask, segment_allowed
from mlx_train_perf_b200.core.loss import (DenseHead, QuantizedHead, fused_linear_ce, linear_cross_entropy,
                                           resolve_impl, tied_head)
from mlx_train_perf_b200.errors import (AttentionInputError, LossInputError, UnsupportedAttentionError,
                                        UnsupportedHeadError)


def _dense(n=4, d=8, v=10, dtype=torch.float32):
    return torch.randn(n, d).to(dtype), DenseHead(weight=torch.randn(v, d).to(dtype)), torch.randint(0, v, (n,))


def test_shape_and_dtype_refusals():
    h, head, t = _dense()
    with pytest.raises(LossInputError, match="2D"):
        linear_cross_entropy(h[0], head, t[0])
    with pytest.raises(LossInputError, match="targets shape"):
        linear_cross_entropy(h, head, t[:2])
    with pytest.raises(LossInputError, match="integer dtype"):
        linear_cross_entropy(h, head, t.float())
    with pytest.raises(LossInputError, match="must match hidden's D"):
        linear_cross_entropy(h, DenseHead(weight=torch.randn(10, 7)), t)
    with pytest.raises(LossInputError, match="must match dense head weight dtype"):
        linear_cross_entropy(h.to(torch.bfloat16), head, t)
    with pytest.raises(LossInputError, match="unknown reduction"):
        linear_cross_entropy(h, head, t, reduction="avg")
    with pytest.raises(LossInputError, match="at least one row"):
        linear_cross_entropy(torch.zeros(0, 8), head, torch.zeros(0, dtype=torch.long))
    with pytest.raises(LossInputError, match="0 <= t < V"):
        linear_cross_entropy(h, head, torch.tensor([0, 1, 2, 10]))
    with pytest.raises(LossInputError, match="CUDA tensor"):
        linear_cross_entropy(h, head, t)          # valid inputs, but on the CPU: no fallback
    with pytest.raises(LossInputError, match="CUDA tensor"):
        fused_linear_ce(h, head, torch.tensor([0, -100, 2, 3]))


def test_resolve_impl():
    _, head, _ = _dense()
    assert resolve_impl(head=head, dtype=torch.float32, n=4, d=8).impl == "simt"
    assert resolve_impl(head=head, dtype=torch.bfloat16, n=4, d=8).impl == "tc"
    assert resolve_impl(head=head, dtype=torch.bfloat16, n=4, d=12).impl == "simt"
    with pytest.raises(UnsupportedHeadError):
        resolve_impl(head=head, dtype=torch.float16, n=4)
    with pytest.raises(UnsupportedHeadError):
        resolve_impl(head=head, dtype=torch.float32, n=4, d=8, impl="tc")
    with pytest.raises(LossInputError):
        resolve_impl(head=head, dtype=torch.float32, n=0)
    with pytest.raises(LossInputError, match="unknown impl"):
        resolve_impl(head=head, dtype=torch.float32, n=4, impl="metal")
    q = QuantizedHead(w_q=torch.zeros(4, 8, dtype=torch.int32), scales=torch.zeros(4, 1), biases=torch.zeros(4, 1))
    assert resolve_impl(head=q, dtype=torch.bfloat16, n=4, d=64).impl == "tc"
    with pytest.raises(UnsupportedHeadError, match="4-bit"):
        resolve_impl(head=QuantizedHead(w_q=q.w_q, scales=q.scales, biases=q.biases, bits=8), dtype=torch.bfloat16, n=4)
    with pytest.raises(UnsupportedHeadError, match="group_size=64"):
        resolve_impl(head=QuantizedHead(w_q=q.w_q, scales=q.scales, biases=q.biases, group_size=32),
                     dtype=torch.bfloat16, n=4)
    w = torch.randn(4, 8, requires_grad=True)
    # a trainable dense head is served (d_weight comes back through autograd); defaults follow the
    # reference: DenseHead trainable, tied_head frozen (core/loss.py:29-48)
    assert resolve_impl(head=DenseHead(weight=w), dtype=torch.float32, n=4).impl == "simt"
    assert DenseHead(weight=w).trainable is True
    assert tied_head(w).trainable is False


def test_attention_gate():
    q = torch.zeros(1, 4, 16, 128, dtype=torch.bfloat16)
    k = torch.zeros(1, 2, 16, 128, dtype=torch.bfloat16)
    assert resolve_attention_impl(q, k, k) == "tc"
    assert resolve_attention_impl(q.float(), k.float(), k.float()) == "simt"
    assert resolve_attention_impl(q[..., :64], k[..., :64], k[..., :64]) == "tc"      # head_dim 64 has its own kernels
    assert resolve_attention_impl(q[..., :64], k[..., :64], k[..., :64], impl="simt") == "simt"
    with pytest.raises(AttentionInputError, match="4-D"):
        resolve_attention_impl(q[0], k, k)
    with pytest.raises(AttentionInputError, match="multiple of Hkv"):
        resolve_attention_impl(q[:, :3], k, k)
    with pytest.raises(AttentionInputError, match="sequence length"):
        resolve_attention_impl(q, k[:, :, :8], k[:, :, :8])
    with pytest.raises(UnsupportedAttentionError, match="head_dim"):
        resolve_attention_impl(q[..., :80], k[..., :80], k[..., :80])
    with pytest.raises(UnsupportedAttentionError, match="causal"):
        resolve_attention_impl(q, k, k, causal=False)
    with pytest.raises(UnsupportedAttentionError, match="fp32/bf16"):
        resolve_attention_impl(q.half(), k.half(), k.half())
    pm = PackedMask(seg_id=torch.zeros(1, 16, dtype=torch.int32), seg_start=torch.zeros(1, 16, dtype=torch.int32))
    with pytest.raises(UnsupportedAttentionError, match="segments"):
        resolve_attention_impl(q, k, k, causal=False, segments=pm)
    with pytest.raises(UnsupportedAttentionError, match="impl='tc'"):
        resolve_attention_impl(q.float(), k.float(), k.float(), impl="tc")


def test_segment_allowed_literal():
    allowed = segment_allowed(torch.tensor([[0, 0, 1, 1]], dtype=torch.int32))
    expected = torch.tensor([[True, False, False, False], [True, True, False, False],
                             [False, False, True, False], [False, False, True, True]])[None, None]
    assert torch.equal(allowed, expected)


def test_operands_on_another_device_are_refused_before_any_native_call():
    """The kernels get raw device addresses, so an lm_head left on the host (offloaded or tied
    embeddings), a k / v on another device or a norm weight elsewhere must be refused by the Python
    surface: as a TMA base pointer it would fault the GPU.  `meta` tensors stand in for "another
    device" here (no GPU is needed to see the refusal, and nothing is launched)."""
    from mlx_train_perf_b200.attention import prestep
    from mlx_train_perf_b200.attention.api import flash_attention
    h = torch.empty(4, 64, dtype=torch.bfloat16, device="meta")
    t = torch.zeros(4, dtype=torch.int64)
    with pytest.raises(LossInputError, match="head.weight is on cpu"):
        linear_cross_entropy(h, DenseHead(weight=torch.zeros(10, 64, dtype=torch.bfloat16)), t, validate_targets=False)
    q_head = QuantizedHead(w_q=torch.zeros(10, 8, dtype=torch.int32), scales=torch.zeros(10, 1, device="meta"),
                           biases=torch.zeros(10, 1, device="meta"))
    with pytest.raises(LossInputError, match="head.w_q is on cpu"):
        fused_linear_ce(h, q_head, t)
    q = torch.empty(1, 4, 16, 128, dtype=torch.bfloat16, device="meta")
    k = torch.zeros(1, 2, 16, 128, dtype=torch.bfloat16)
    with pytest.raises(AttentionInputError, match="one device"):
        flash_attention(q, k, k, scale=1.0)
    with pytest.raises(AttentionInputError, match="one device"):
        flash_attention(k.repeat(1, 2, 1, 1), q[:, :2], k, scale=1.0)
    x = torch.empty(1, 16, 4, 128, dtype=torch.bfloat16, device="cpu")
    cs = torch.zeros(16, 128)
    with pytest.raises(AttentionInputError, match="CUDA"):
        prestep.qk_norm_rope(x, cs, cs)


def test_segment_contract_validator():
    """`validate_segments=True` checks what the tensor-core kernels assume about a PackedMask: ids
    start at 0, never decrease or skip, and seg_start is the first index of the row's segment."""
    from mlx_train_perf_b200.attention.api import check_segment_contract
    ok_id = torch.tensor([[0, 0, 0, 1, 1, 2]], dtype=torch.int32)
    ok_st = torch.tensor([[0, 0, 0, 3, 3, 5]], dtype=torch.int32)
    check_segment_contract(ok_id, ok_st)
    for bad_id, bad_st in (
            (torch.tensor([[1, 1, 1, 2, 2, 3]]), ok_st),                 # does not start at 0
            (torch.tensor([[0, 0, 1, 0, 0, 2]]), ok_st),                 # decreases
            (torch.tensor([[0, 0, 0, 2, 2, 3]]), ok_st),                 # skips an id
            (ok_id, torch.tensor([[0, 0, 0, 2, 2, 5]])),                 # start is not the segment's first index
            (ok_id, torch.tensor([[0, 1, 2, 3, 4, 5]]))):
        with pytest.raises(AttentionInputError, match="PackedMask contract"):
            check_segment_contract(bad_id.to(torch.int32), bad_st.to(torch.int32))


def test_aliasing_views_are_detected():
    """The backward writes dQ / dK / dV through the input strides: a view whose elements alias (k
    expanded over the GQA group or the batch) must be copied first, a permuted projection must not."""
    from mlx_train_perf_b200.attention.api import _inner_contig, _non_overlapping
    base = torch.zeros(2, 16, 4, 64)                        # (B, N, H, D) projection
    assert _non_overlapping(base.permute(0, 2, 1, 3))       # consumed in place
    assert _non_overlapping(base.permute(0, 2, 1, 3)[:, :, ::2])
    k = torch.zeros(1, 1, 16, 64)
    assert not _non_overlapping(k.expand(1, 4, 16, 64))     # heads alias
    assert not _non_overlapping(k.expand(3, 1, 16, 64))     # batches alias
    assert _inner_contig(k.expand(1, 4, 16, 64)).is_contiguous()
    assert not _non_overlapping(torch.zeros(1, 2, 16, 128)[..., ::2])   # head_dim stride 2


def test_masked_loss_refuses_host_tensors():
    """`masked_loss` hands raw addresses to two library kernels: host tensors never get that far."""
    from mlx_train_perf_b200.core.loss import masked_loss
    with pytest.raises(LossInputError, match="CUDA"):
        masked_loss(torch.zeros(4), torch.zeros(4, dtype=torch.int64))
