"""Generation: sampling filters, and KV-cached decoding against full re-computation (CPU)."""

import pytest
import torch

from olmo_core_b200.generate import GenerationConfig, TransformerGenerationModule
from olmo_core_b200.generate.sampling import select_next_token, top_k_filtering, top_p_filtering
from olmo_core_b200.generate.utils import selective_log_softmax
from olmo_core_b200.nn.transformer import TransformerConfig


def test_filters():
    logits = torch.tensor([[1.0, 3.0, 2.0, 0.0]])
    assert top_k_filtering(logits, 2).isinf().tolist() == [[True, False, False, True]]
    probs = torch.softmax(logits, -1)
    kept = ~top_p_filtering(logits, float(probs[0, 1]) + 1e-3).isinf()
    assert kept.tolist() == [[False, True, True, False]]  # the token that crosses the threshold stays
    assert select_next_token(logits, do_sample=False).item() == 1
    assert select_next_token(logits, temperature=0.0).item() == 1
    torch.manual_seed(0)
    draws = torch.stack([select_next_token(logits.repeat(64, 1), temperature=1.0, top_k=2) for _ in range(4)])
    assert set(draws.unique().tolist()) <= {1, 2}
    lp = selective_log_softmax(logits, torch.tensor([1]))
    torch.testing.assert_close(lp, torch.log_softmax(logits, -1)[:, 1])


@pytest.mark.parametrize("left_pad", [False, True])
def test_cached_decoding_matches_recomputation(left_pad):
    torch.manual_seed(0)
    model = TransformerConfig.olmo2_30M(vocab_size=128, n_layers=2).build(init_device="cpu")
    model.init_weights(max_seq_len=64, device=torch.device("cpu"))
    gen = TransformerGenerationModule(model, GenerationConfig(pad_token_id=0, eos_token_id=1, max_new_tokens=6, do_sample=False),
                                      device=torch.device("cpu"))
    ids = torch.randint(2, 128, (2, 8))
    mask = None
    if left_pad:
        ids[0, :3] = 0
        mask = torch.ones_like(ids, dtype=torch.bool)
        mask[0, :3] = False
    cached, _, lp = gen.generate_batch(ids, attention_mask=mask, return_logprobs=True, log_timing=False)
    assert cached.shape == (2, 14) and lp.shape == (2, 6)
    if not left_pad:
        plain, _, _ = gen.generate_batch(ids, use_cache=False, max_length=14, log_timing=False)
        assert torch.equal(cached, plain)
    else:
        # the padded sequence must continue exactly like its unpadded self
        alone, _, _ = gen.generate_batch(ids[:1, 3:], log_timing=False)
        assert torch.equal(cached[0, 3:], alone[0])
