"""``generate_step``, the token-level generator under ``stream_generate`` (mlx_lm/generate.py:298-462)."""
import pytest
import torch

from helpers import CONFIG_B, make_model_dir, random_tokens

pytestmark = pytest.mark.gpu


def test_generate_step_yields_tokens_and_their_log_probabilities(tmp_path):
    """Token ids in, (token, log-probability vector) out; with the greedy sampler the token is the vector's
    best entry, the vector is normalised, the prompt's progress is reported portion by portion, and the tokens
    are those of ``stream_generate`` cut the same way."""
    from mlx_lm_b200 import generate_step, load, stream_generate

    make_model_dir(str(tmp_path), dict(CONFIG_B), 3, peaky=10.0)
    model, tokenizer = load(str(tmp_path), dtype="float32")
    vocab = CONFIG_B["vocab_size"]
    prompt = random_tokens(11, vocab, 4)
    seen = []
    pairs = list(generate_step(torch.tensor(prompt), model, max_tokens=9, prefill_step_size=4,
                               prompt_progress_callback=lambda done, total: seen.append((done, total))))
    assert len(pairs) == 9
    for token, logprobs in pairs:
        assert logprobs.shape == (vocab,) and logprobs.dtype == torch.float32
        assert int(logprobs.argmax()) == token
        assert abs(float(logprobs.exp().sum()) - 1.0) < 1e-4
    assert seen == [(4, 11), (8, 11), (11, 11)]
    streamed = [r.token for r in stream_generate(model, tokenizer, prompt, max_tokens=9, prefill_step_size=4)]
    assert [t for t, _ in pairs] == streamed
