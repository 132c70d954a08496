"""Host logic of the module-level replacement (no GPU): which modules are swapped, what is shared, what is refused."""

import pytest
import torch

from fa4b.lowp_module import LowpFA4Attention, pair_interleave_qk_rows, replace_attention_modules


class _Attention(torch.nn.Module):  # the attributes of TorchTitan's Llama Attention that the replacement reads
    def __init__(self, hidden=512, n_heads=4, n_kv_heads=2, head_dim=128, dtype=torch.bfloat16):
        super().__init__()
        self.n_heads, self.n_kv_heads, self.head_dim = n_heads, n_kv_heads, head_dim
        self.wq = torch.nn.Linear(hidden, n_heads * head_dim, bias=False, dtype=dtype)
        self.wk = torch.nn.Linear(hidden, n_kv_heads * head_dim, bias=False, dtype=dtype)
        self.wv = torch.nn.Linear(hidden, n_kv_heads * head_dim, bias=False, dtype=dtype)
        self.wo = torch.nn.Linear(n_heads * head_dim, hidden, bias=False, dtype=dtype)


class _Layer(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.attention = _Attention()
        self.feed_forward = torch.nn.Linear(512, 512, dtype=torch.bfloat16)


def test_replacement_shares_the_projections_and_keeps_state_dict_keys():
    model = torch.nn.ModuleDict({"layers": torch.nn.ModuleList([_Layer(), _Layer()])})
    keys = set(model.state_dict().keys())
    originals = [layer.attention for layer in model["layers"]]
    assert replace_attention_modules(model) == 2
    for layer, orig in zip(model["layers"], originals):
        assert isinstance(layer.attention, LowpFA4Attention)
        assert layer.attention.wq is orig.wq and layer.attention.wo is orig.wo
        assert (layer.attention.n_heads, layer.attention.n_kv_heads, layer.attention.head_dim) == (4, 2, 128)
    assert set(model.state_dict().keys()) == keys
    assert replace_attention_modules(model) == 0  # idempotent


def test_replacement_refuses_what_it_cannot_run():
    with pytest.raises(TypeError):
        LowpFA4Attention.from_attention(torch.nn.Linear(4, 4))
    with pytest.raises(TypeError):
        LowpFA4Attention.from_attention(_Attention(dtype=torch.float32))
    biased = _Attention()
    biased.wq = torch.nn.Linear(512, 512, bias=True, dtype=torch.bfloat16)
    with pytest.raises(TypeError):
        LowpFA4Attention.from_attention(biased)
    mod = LowpFA4Attention.from_attention(_Attention())
    with pytest.raises(ValueError):
        mod(torch.zeros(1, 128, 512, dtype=torch.bfloat16), (None, None), attention_masks=object())
    with pytest.raises(TypeError):
        mod._rope_tables(torch.zeros(4, 4))


def test_complex_freqs_become_bf16_tables_once():
    mod = LowpFA4Attention.from_attention(_Attention())
    ang = torch.arange(8, dtype=torch.float32)[:, None] * torch.tensor([1.0, 0.1])[None, :]
    freqs = torch.polar(torch.ones_like(ang), ang)
    cos, sin = mod._rope_tables(freqs)
    assert cos.dtype == torch.bfloat16 and cos.shape == (8, 2)
    assert torch.equal(cos, ang.cos().bfloat16()) and torch.equal(sin, ang.sin().bfloat16())
    assert mod._rope_tables(freqs)[0] is cos  # cached


def test_pair_interleave_is_a_per_head_permutation():
    w = torch.arange(2 * 8 * 3, dtype=torch.float32).reshape(16, 3)
    wi = pair_interleave_qk_rows(w, 2, 8)
    assert sorted(wi[:, 0].tolist()) == sorted(w[:, 0].tolist())
    assert torch.equal(wi[:8][0::2], w[:4]) and torch.equal(wi[:8][1::2], w[4:8])
