"""Options without a device: the command line has mlx-lm's names and defaults (mlx_lm/generate.py:36-46, 54-213),
the samplers and logits processors refuse what mlx-lm refuses (mlx_lm/sample_utils.py:142-146, 175-182, 256-263),
and their records for the sampling kernel are what csrc/sampling.cu's structs expect."""
import struct

import pytest

from mlx_lm_b200.sampling import GREEDY, LogitsProcessors, Sampler, make_logits_processors, make_sampler


def test_command_line_names_and_defaults():
    import importlib

    G = importlib.import_module("mlx_lm_b200.generate")
    a = G.setup_arg_parser().parse_args([])
    assert (a.prompt, a.max_tokens, a.temp, a.top_p, a.min_p, a.top_k) == ("hello", 100, 0.0, 1.0, 0.0, 0)
    assert (a.xtc_probability, a.xtc_threshold, a.min_tokens_to_keep, a.seed) == (0.0, 0.1, 1, None)   # mlx_lm/generate.py:124-128
    assert a.verbose is True and a.ignore_chat_template is False and a.model is None
    assert a.dtype == "bfloat16" and a.page_size == 16 and a.prefill_step_size == 2048
    b = G.setup_arg_parser().parse_args(["--model", "m", "-p", "5 6", "-m", "7", "--temp", "0.5", "--top-p", "0.9",
                                         "--min-p", "0.05", "--top-k", "40", "--xtc-probability", "0.3",
                                         "--xtc-threshold", "0.2", "--min-tokens-to-keep", "2", "--seed", "11",
                                         "--extra-eos-token", "3", "4", "--verbose", "F", "--ignore-chat-template"])
    assert (b.model, b.prompt, b.max_tokens, b.temp, b.top_p, b.min_p, b.top_k) == ("m", "5 6", 7, 0.5, 0.9, 0.05, 40)
    assert (b.xtc_probability, b.xtc_threshold, b.min_tokens_to_keep, b.seed) == (0.3, 0.2, 2, 11)
    assert list(b.extra_eos_token) == ["3", "4"] and b.verbose is False and b.ignore_chat_template is True
    assert G.str2bool("T") and G.str2bool("true") and not G.str2bool("F")


def test_sampler_options_and_what_is_refused():
    assert make_sampler() == GREEDY == Sampler()                 # temp 0: greedy, whatever else is set
    assert make_sampler(temp=0.0, top_p=0.5, top_k=3) == GREEDY
    s = make_sampler(temp=0.8, top_p=0.95, min_p=0.1, min_tokens_to_keep=2, top_k=50, xtc_probability=0.5,
                     xtc_threshold=0.1, xtc_special_tokens=[1, 2], seed=9)
    assert (s.temp, s.top_p, s.min_p, s.min_tokens_to_keep, s.top_k) == (0.8, 0.95, 0.1, 2, 50)
    assert (s.xtc_probability, s.xtc_threshold, s.xtc_special_tokens, s.seed) == (0.5, 0.1, (1, 2), 9)
    for bad in (dict(temp=-1.0), dict(temp=1.0, min_p=1.5), dict(temp=1.0, min_tokens_to_keep=0),
                dict(temp=1.0, top_k=-1), dict(temp=1.0, top_k=1.5), dict(temp=1.0, xtc_threshold=0.6),
                dict(temp=1.0, xtc_probability=1.5), dict(temp=1.0, xtc_special_tokens=list(range(65)))):
        with pytest.raises(ValueError):
            make_sampler(**bad)


def test_sampler_record_for_the_kernel():
    s = make_sampler(temp=0.7, top_p=0.9, min_p=0.05, min_tokens_to_keep=3, top_k=40, xtc_probability=0.25,
                     xtc_threshold=0.2)
    rec = s.words(seed=(5 << 32) | 6, request=1234, position=77)
    assert len(rec) == 16 * 4
    temp, top_p, min_p, xp, xt, top_k, keep, lo, hi, req, pos, *pad = struct.unpack("<5f2i4I5i", rec)
    assert (round(temp, 6), round(top_p, 6), round(min_p, 6), round(xp, 6), round(xt, 6)) == (0.7, 0.9, 0.05, 0.25, 0.2)
    assert (top_k, keep, lo, hi, req, pos) == (40, 3, 6, 5, 1234, 77) and pad == [0] * 5
    # a sampler with a seed of its own ignores the scheduler's; the draw is keyed by (seed, request, position)
    own = make_sampler(temp=1.0, seed=3).words(seed=99, request=1, position=2)
    assert struct.unpack("<5f2i4I5i", own)[7:11] == (3, 0, 1, 2)
    assert s.words(1, 2, 3) == s.words(1, 2, 3) != s.words(1, 2, 4)


def test_logits_processors_options_and_record():
    assert make_logits_processors() == [] and make_logits_processors(repetition_penalty=0.0) == []
    (p,) = make_logits_processors(logit_bias={7: -1.5, 3: 2.0}, repetition_penalty=1.2, repetition_context_size=30,
                                  presence_penalty=0.4, frequency_penalty=0.1, frequency_context_size=10)
    assert isinstance(p, LogitsProcessors) and dict(p.logit_bias) == {7: -1.5, 3: 2.0}
    assert p.context_size == 30                                   # the longest window of the penalties in use
    assert make_logits_processors(presence_penalty=0.5)[0].context_size == 20
    rep, pres, freq, rc, pc, fc, n_bias, pad = struct.unpack("<3f5i", p.words())
    assert (round(rep, 6), round(pres, 6), round(freq, 6), rc, pc, fc, n_bias, pad) == (1.2, 0.4, 0.1, 30, 20, 10, 2, 0)
    with pytest.raises(ValueError):
        make_logits_processors(repetition_penalty=-1.0)
    with pytest.raises(ValueError):
        make_logits_processors(repetition_penalty="high")
