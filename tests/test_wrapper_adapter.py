"""`enable_flash_attention` and the trainer loss shims on tiny synthetic Hugging-Face models
(random init, no checkpoint): enable-time refusals and module-tree contract on CPU
(tests/test_attention_wrapper.py of the reference), forward/backward parity against the stock
eager attention and packed-vs-unpacked loss agreement on the GPU
(tests/test_adapter_packed.py:13-40 pins packed vs unpacked loss <= 2e-2)."""
import copy

import pytest
import torch

from mlx_train_perf_b200.adapters.torch_lm import make_loss_fn, make_packed_loss_fn, split_model
from mlx_train_perf_b200.attention.segments import PackedMask
from mlx_train_perf_b200.attention.wrapper import FlashAttentionWrapper, _resolve_mask, enable_flash_attention
from mlx_train_perf_b200.data.packing import build_row
from mlx_train_perf_b200.errors import AdapterError, AttentionInputError, UnsupportedAttentionError

transformers = pytest.importorskip("transformers")


def _tiny(family="llama", **over):
    kw = dict(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, max_position_embeddings=512, attention_dropout=0.0)
    kw.update(over)
    torch.manual_seed(0)
    if family == "llama":
        m = transformers.LlamaForCausalLM(transformers.LlamaConfig(**kw))
    elif family == "qwen3":
        m = transformers.Qwen3ForCausalLM(transformers.Qwen3Config(head_dim=64, **kw))
    else:
        m = transformers.Qwen2ForCausalLM(transformers.Qwen2Config(**kw))
    m.lm_head.weight.requires_grad_(False)      # LoRA-style: the head is frozen
    return m


def test_enable_swaps_every_layer_and_keeps_module_paths():
    m = _tiny("qwen3")
    names_before = {n for n, _ in m.named_parameters()}
    enable_flash_attention(m)
    assert all(isinstance(layer.self_attn, FlashAttentionWrapper) for layer in m.model.layers)
    assert {n for n, _ in m.named_parameters()} == names_before      # q_proj ... q_norm paths survive
    w = m.model.layers[0].self_attn
    assert (w.n_heads, w.n_kv_heads, w.head_dim, w.scale) == (4, 2, 64, 0.125) and w._has_qk_norm
    enable_flash_attention(m)                                          # idempotent
    assert isinstance(m.model.layers[0].self_attn.q_proj, torch.nn.Linear)


def test_enable_time_refusals():
    with pytest.raises(UnsupportedAttentionError, match="dropout"):
        enable_flash_attention(_tiny(attention_dropout=0.1))
    with pytest.raises(UnsupportedAttentionError, match="head_dim"):
        enable_flash_attention(_tiny(hidden_size=160, num_attention_heads=4))      # head_dim 40
    gpt = transformers.GPT2LMHeadModel(transformers.GPT2Config(n_layer=1, n_head=2, n_embd=64, vocab_size=100))
    with pytest.raises(UnsupportedAttentionError, match="unsupported model architecture"):
        enable_flash_attention(gpt)
    q2 = _tiny("qwen2")
    q2.config.layer_types = ["full_attention", "sliding_attention"]
    with pytest.raises(UnsupportedAttentionError, match="layer_types"):
        enable_flash_attention(q2)
    with pytest.raises(AdapterError, match="unsupported model architecture"):
        split_model(gpt)
    with pytest.raises(AdapterError, match="enable_flash_attention"):
        make_packed_loss_fn(_tiny())


def test_mask_contract():
    pm = PackedMask(seg_id=torch.zeros(1, 4, dtype=torch.int32), seg_start=torch.zeros(1, 4, dtype=torch.int32))
    assert _resolve_mask(None) is True and _resolve_mask("causal") is True and _resolve_mask(pm) is pm
    with pytest.raises(AttentionInputError, match="string mask"):
        _resolve_mask("sliding")
    with pytest.raises(AttentionInputError, match="tensor attention masks"):
        _resolve_mask(torch.zeros(1, 1, 4, 4))
    m = _tiny()
    enable_flash_attention(m)
    with pytest.raises(AttentionInputError, match="KV cache"):
        m.model.layers[0].self_attn(torch.zeros(1, 4, 256), past_key_values=object())


@pytest.mark.gpu
@pytest.mark.parametrize("family", ["llama", "qwen2", "qwen3"])
def test_wrapped_model_matches_stock_eager(cuda_device, family):
    dev = cuda_device
    stock = _tiny(family).to(dev).float()
    stock.config._attn_implementation = "eager"
    ours = copy.deepcopy(stock)
    enable_flash_attention(ours)
    torch.manual_seed(1)
    batch = torch.randint(1, 512, (2, 97), device=dev)
    lengths = torch.tensor([[1, 96], [5, 60]], device=dev)
    loss, ntoks = make_loss_fn(ours)(ours, batch, lengths)
    loss.backward()
    logits = stock(batch[:, :-1]).logits.float()
    steps = torch.arange(1, 97, device=dev)
    mask = (steps >= lengths[:, 0:1]) & (steps <= lengths[:, 1:2])
    nll = torch.nn.functional.cross_entropy(logits.reshape(-1, 512), batch[:, 1:].reshape(-1), reduction="none")
    ref = (nll.reshape(2, 96) * mask).sum() / mask.sum()
    ref.backward()
    assert int(ntoks) == int(mask.sum())
    assert abs(loss.item() - ref.item()) < 1e-4 * max(1.0, abs(ref.item()))
    g_ours = ours.model.layers[0].self_attn.q_proj.weight.grad
    g_ref = stock.model.layers[0].self_attn.q_proj.weight.grad
    assert (g_ours - g_ref).abs().max().item() < 1e-3 * max(1e-6, g_ref.abs().max().item()) + 1e-7
    g_ours = ours.model.embed_tokens.weight.grad
    g_ref = stock.model.embed_tokens.weight.grad
    assert (g_ours - g_ref).abs().max().item() < 1e-3 * g_ref.abs().max().item() + 1e-7


@pytest.mark.gpu
def test_full_finetune_head_gradient(cuda_device):
    """An lm_head that requires grad (full fine-tune) gets its gradient from the fused loss
    (the reference's trainable-head path, core/loss.py:234-267)."""
    dev = cuda_device
    stock = _tiny("llama").to(dev).float()
    stock.lm_head.weight.requires_grad_(True)
    stock.config._attn_implementation = "eager"
    ours = copy.deepcopy(stock)
    enable_flash_attention(ours)
    torch.manual_seed(3)
    batch = torch.randint(1, 512, (2, 65), device=dev)
    lengths = torch.tensor([[1, 64], [1, 64]], device=dev)
    loss, _ = make_loss_fn(ours)(ours, batch, lengths)
    loss.backward()
    logits = stock(batch[:, :-1]).logits.float()
    ref = torch.nn.functional.cross_entropy(logits.reshape(-1, 512), batch[:, 1:].reshape(-1))
    ref.backward()
    g_ours, g_ref = ours.lm_head.weight.grad, stock.lm_head.weight.grad
    assert g_ours is not None
    assert (g_ours - g_ref).abs().max().item() < 1e-3 * g_ref.abs().max().item() + 1e-7


@pytest.mark.gpu
def test_packed_loss_matches_unpacked(cuda_device):
    dev = cuda_device
    m = _tiny("llama", max_position_embeddings=256).to(dev).float()
    enable_flash_attention(m)
    torch.manual_seed(2)
    seqs = [torch.randint(1, 512, (n,)).tolist() for n in (40, 25, 33)]
    row, sid, sst, lmask = build_row([(s, 0) for s in seqs], 128)
    t = lambda x, dt: torch.tensor([x], dtype=dt, device=dev)
    ploss, pn = make_packed_loss_fn(m)(m, t(row, torch.int64), t(sid, torch.int32), t(sst, torch.int32),
                                       t(lmask, torch.bool))
    # unpacked: each sequence alone; note packed positions are not reset, so RoPE phases differ
    # (relative-position invariance keeps the attention identical up to rounding)
    tot, cnt = 0.0, 0
    unpacked = make_loss_fn(m)
    for s in seqs:
        b = torch.tensor([s + [0]], device=dev)
        l, n = unpacked(m, b, torch.tensor([[1, len(s)]], device=dev))   # steps 1..n, the packed window
        tot += l.item() * int(n)
        cnt += int(n)
    assert int(pn) == cnt
    assert abs(ploss.item() - tot / cnt) < 2e-2
