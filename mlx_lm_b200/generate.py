"""Entry points in mlx-lm's manner: ``load``, ``generate``, ``stream_generate``,
``batch_generate``, ``BatchGenerator`` and the ``generate`` command line
(mlx_lm/generate.py:54-213, 648-790, 1565-2060, 2063-2186; ``load`` is
mlx_lm/utils.py:483-541).  Names and meanings of options follow mlx-lm where
it has them; what this engine does not build (adapters, draft models,
quantized caches, chat templates, prompt-cache files) is not offered.

All generation, single or batched, runs through one ``Scheduler`` over one
``Engine``: a single request is a batch of one.
"""

from __future__ import annotations

import argparse
import contextlib
import json
import sys
import time
from dataclasses import dataclass
from typing import Any, Callable, Dict, Generator, List, Optional, Sequence, Tuple, Union

import torch

from .engine.scheduler import PromptProgress, Response, Scheduler, StopSequenceMatcher
from .engine.step import Engine
from .sampling import GREEDY, Sampler, make_logits_processors, make_sampler
from .sampling.device import DeviceSampler
from .tokenizer_utils import TokenizerWrapper, load_tokenizer
from .weights import load_model

DEFAULT_PROMPT = "hello"
DEFAULT_MAX_TOKENS = 100
DEFAULT_TEMP = 0.0
DEFAULT_TOP_P = 1.0
DEFAULT_MIN_P = 0.0
DEFAULT_TOP_K = 0
DEFAULT_XTC_PROBABILITY = 0.0
DEFAULT_XTC_THRESHOLD = 0.1    # the command line's default (mlx_lm/generate.py:124-128)
DEFAULT_MIN_TOKENS_TO_KEEP = 1
DEFAULT_SEED = None


# ---------------------------------------------------------------------- loading

def load(path: str, tokenizer_config: Optional[dict] = None, model_config: Optional[dict] = None,
         adapter_path: Optional[str] = None, lazy: bool = False, return_config: bool = False,
         revision: Optional[str] = None, trust_remote_code: bool = False, dtype: str = "bfloat16",
         device: str = "cuda"):
    """Model folder -> ``(model, tokenizer)`` (or ``(model, tokenizer, config)``), the signature of
    mlx-lm's ``load`` (mlx_lm/utils.py:483-541).

    Local folders only (``revision`` and ``trust_remote_code`` are accepted and unused; ``adapter_path``
    must be None: adapters are not built).  ``dtype`` is ``"bfloat16"`` (the serving path) or
    ``"float32"`` (everything in true 32-bit).  ``tokenizer_config`` may carry ``eos_token_ids``."""
    if adapter_path is not None:
        raise ValueError("adapter_path: adapters are not offered by this engine")
    model, config = load_model(path, dtype=dtype, device=device, model_config=model_config)
    tokenizer = load_tokenizer(path, config, (tokenizer_config or {}).get("eos_token_ids"))
    return (model, tokenizer, config) if return_config else (model, tokenizer)


def get_engine(model, page_size: int = 16, num_pages: Optional[int] = None, max_requests: int = 64) -> Engine:
    """The engine of a model, made on first use and kept on the model (the page pool is allocated once)."""
    key = (page_size, num_pages, max_requests)
    cache = model.__dict__.setdefault("_engines", {})
    if key not in cache:
        cache.clear()    # one pool at a time: the old one is freed before the new one is made
        cache[key] = Engine(model, page_size=page_size, n_pages=num_pages, max_requests=max_requests)
    return cache[key]


# ---------------------------------------------------------------------- single stream

@dataclass
class GenerationResponse:
    """What ``stream_generate`` yields (mlx_lm/generate.py:260-287).  ``logprobs`` is the
    log-probability of ``token``, or the whole float32 ``[vocab]`` vector (a CUDA tensor) when
    ``return_logprobs=True`` was asked for."""
    text: str
    token: int
    logprobs: Any
    from_draft: bool
    prompt_tokens: int
    prompt_tps: float
    generation_tokens: int
    generation_tps: float
    peak_memory: float
    finish_reason: Optional[str] = None


def _encode(tokenizer: TokenizerWrapper, prompt) -> List[int]:
    if isinstance(prompt, str):
        add = tokenizer.bos_token is None or not prompt.startswith(tokenizer.bos_token)
        return tokenizer.encode(prompt, add_special_tokens=add)
    if isinstance(prompt, torch.Tensor):
        return [int(t) for t in prompt.flatten().tolist()]
    return [int(t) for t in prompt]


def stream_generate(model, tokenizer: TokenizerWrapper, prompt: Union[str, List[int], torch.Tensor],
                    max_tokens: int = 256, sampler: Optional[Sampler] = None,
                    logits_processors: Optional[Sequence] = None, prefill_step_size: int = 2048,
                    prompt_progress_callback: Optional[Callable[[int, int], None]] = None,
                    seed: Optional[int] = None, return_logprobs: bool = False, engine: Optional[Engine] = None,
                    ) -> Generator[GenerationResponse, None, None]:
    """Yield the generated text segment by segment.  Stops at an end-of-sequence token
    (``finish_reason="stop"``, the token is not part of the text) or after ``max_tokens``
    (``"length"``); the last response carries the reason.  ``seed=None``: a fresh seed for every call."""
    tokens = _encode(tokenizer, prompt)
    engine = engine or get_engine(model)
    dev_sampler = DeviceSampler(model.device, seed=seed, return_logprobs=return_logprobs, engine=engine)
    sched = Scheduler(engine, dev_sampler, max_requests=1, max_prefilling=1, prefill_step_size=prefill_step_size,
                      max_tokens_per_step=max(prefill_step_size, 1))
    stop = StopSequenceMatcher([[t] for t in tokenizer.eos_token_ids])
    uid = sched.insert(tokens, max_tokens, sampler or GREEDY, logits_processors or (), stop)
    detok = tokenizer.detokenizer
    torch.cuda.reset_peak_memory_stats(model.device)
    tic = time.perf_counter()
    prompt_tps, n = 0.0, 0
    try:
        while sched.has_work():
            progress, responses = sched.next()
            if prompt_progress_callback is not None:
                for p in progress:
                    prompt_progress_callback(*p.progress)
            for r in responses:
                if r.finish_reason == "cancelled":
                    continue
                if n == 0:
                    prompt_tps = len(tokens) / max(time.perf_counter() - tic, 1e-9)
                    tic = time.perf_counter()
                n += 1
                if r.finish_reason != "stop":
                    detok.add_token(r.token)
                if r.finish_reason is not None:
                    detok.finalize()
                lp = dev_sampler.last_logprobs[0].clone() if return_logprobs else r.logprobs
                yield GenerationResponse(detok.last_segment, r.token, lp, False, len(tokens), prompt_tps, n,
                                         n / max(time.perf_counter() - tic, 1e-9),
                                         torch.cuda.max_memory_allocated(model.device) / 1e9, r.finish_reason)
    finally:
        sched.remove([uid])


def generate_step(prompt: Union[List[int], torch.Tensor], model, *, max_tokens: int = 256,
                  sampler: Optional[Sampler] = None, logits_processors: Optional[Sequence] = None,
                  prefill_step_size: int = 2048,
                  prompt_progress_callback: Optional[Callable[[int, int], None]] = None,
                  seed: Optional[int] = None,
                  engine: Optional[Engine] = None) -> Generator[Tuple[int, torch.Tensor], None, None]:
    """Token ids in, ``(token, log-probabilities)`` out, one pair per generated token
    (mlx_lm/generate.py:298-462): the log-probabilities are the float32 ``[vocab]`` vector the token was drawn
    from, on the device.  No tokenizer and no end-of-sequence token: it stops after ``max_tokens``."""
    tokens = [int(t) for t in (prompt.flatten().tolist() if isinstance(prompt, torch.Tensor) else prompt)]
    engine = engine or get_engine(model)
    dev_sampler = DeviceSampler(model.device, seed=seed, return_logprobs=True, engine=engine)
    sched = Scheduler(engine, dev_sampler, max_requests=1, max_prefilling=1, prefill_step_size=prefill_step_size,
                      max_tokens_per_step=max(prefill_step_size, 1))
    uid = sched.insert(tokens, max_tokens, sampler or GREEDY, logits_processors or ())
    try:
        while sched.has_work():
            progress, responses = sched.next()
            if prompt_progress_callback is not None:
                for p in progress:
                    prompt_progress_callback(*p.progress)
            for r in responses:
                if r.finish_reason != "cancelled":
                    yield r.token, dev_sampler.last_logprobs[0].clone()
    finally:
        sched.remove([uid])


def generate(model, tokenizer, prompt: Union[str, List[int]], verbose: bool = False, **kwargs) -> str:
    """The whole response as one string; ``verbose`` prints it as it comes, then speeds and memory."""
    if verbose:
        print("=" * 10)
    text = ""
    response = None
    for response in stream_generate(model, tokenizer, prompt, **kwargs):
        if verbose:
            print(response.text, end="", flush=True)
        text += response.text
    if verbose:
        print()
        print("=" * 10)
        if response is None or len(text) == 0:
            print("No text generated for this prompt")
            return text
        print(f"Prompt: {response.prompt_tokens} tokens, {response.prompt_tps:.3f} tokens-per-sec")
        print(f"Generation: {response.generation_tokens} tokens, {response.generation_tps:.3f} tokens-per-sec")
        print(f"Peak memory: {response.peak_memory:.3f} GB")
    return text


# ---------------------------------------------------------------------- batches

@dataclass
class BatchStats:
    prompt_tokens: int = 0
    prompt_tps: float = 0
    prompt_time: float = 0
    generation_tokens: int = 0
    generation_tps: float = 0
    generation_time: float = 0
    peak_memory: float = 0


@dataclass
class BatchResponse:
    texts: List[str]
    stats: BatchStats
    caches: Optional[List[Any]] = None
    token_ids: Optional[List[List[int]]] = None
    logprobs: Optional[List[List[float]]] = None


class BatchGenerator:
    """Continuous batching with mlx-lm's surface (mlx_lm/generate.py:1565-1945).

    ``completion_batch_size`` bounds the requests that run at once, ``prefill_batch_size`` those of
    them still in their prompt, ``prefill_step_size`` the portion of one prompt per step; added
    here: ``max_tokens_per_step`` (token budget of a step), ``seed``, and the pool's ``page_size``
    / ``num_pages``.  Prompt caches cannot be passed in or handed out (``caches`` must be None)."""

    Response = Response

    def __init__(self, model, *, max_tokens: int = 128, stop_tokens: Optional[Sequence[Sequence[int]]] = None,
                 sampler: Optional[Sampler] = None, logits_processors: Optional[Sequence] = None,
                 completion_batch_size: int = 32, prefill_batch_size: int = 8, prefill_step_size: int = 2048,
                 max_kv_size: Optional[int] = None, stream=None, max_tokens_per_step: Optional[int] = None,
                 seed: Optional[int] = None, page_size: int = 16, num_pages: Optional[int] = None,
                 engine: Optional[Engine] = None, return_logprobs: bool = False):
        if max_kv_size is not None:
            raise ValueError("max_kv_size (a rotating cache for the whole run) is not offered: which keys a layer "
                             "keeps is a property of its mixer (a window), not an option of a run")
        self.model = model
        self.max_tokens = max_tokens
        self.sampler = sampler or GREEDY
        self.logits_processors = tuple(logits_processors or ())
        self.completion_batch_size = max(completion_batch_size, prefill_batch_size)
        self.prefill_batch_size, self.prefill_step_size = prefill_batch_size, prefill_step_size
        self.engine = engine or get_engine(model, page_size=page_size, num_pages=num_pages,
                                           max_requests=max(64, self.completion_batch_size))
        self._sampler = DeviceSampler(model.device, seed=seed, return_logprobs=return_logprobs, engine=self.engine)
        self._sched = Scheduler(self.engine, self._sampler, max_requests=self.completion_batch_size,
                                max_prefilling=prefill_batch_size, prefill_step_size=prefill_step_size,
                                max_tokens_per_step=max_tokens_per_step or max(prefill_step_size, 1))
        self._default_stop = StopSequenceMatcher(stop_tokens)
        self._prompt_time = 0.0
        self._prompt_tokens = 0
        self._gen_tokens = 0

    def close(self) -> None:
        self._sched.remove([r.uid for r in list(self._sched.running)] + [r.uid for r in self._sched.waiting])

    @contextlib.contextmanager
    def stats(self, stats: Optional[BatchStats] = None):
        stats = stats or BatchStats()
        self._prompt_time = 0.0
        self._prompt_tokens = self._gen_tokens = 0
        torch.cuda.reset_peak_memory_stats(self.model.device)
        tic = time.perf_counter()
        try:
            yield stats
        finally:
            total = time.perf_counter() - tic
            stats.prompt_tokens += self._prompt_tokens
            stats.prompt_time += self._prompt_time
            stats.prompt_tps = stats.prompt_tokens / max(stats.prompt_time, 1e-9)
            stats.generation_tokens += self._gen_tokens
            stats.generation_time += total - self._prompt_time
            stats.generation_tps = stats.generation_tokens / max(stats.generation_time, 1e-9)
            stats.peak_memory = max(stats.peak_memory, torch.cuda.max_memory_allocated(self.model.device) / 1e9)

    def insert(self, prompts: List[List[int]], max_tokens: Optional[List[int]] = None, caches=None,
               all_tokens=None, samplers: Optional[List[Optional[Sampler]]] = None,
               logits_processors: Optional[List[Sequence]] = None,
               stop_matchers: Optional[List[StopSequenceMatcher]] = None) -> List[int]:
        if caches is not None and any(c is not None for c in caches):
            raise ValueError("prompt caches cannot be passed in: requests start from an empty cache")
        n = len(prompts)
        max_tokens = max_tokens or [self.max_tokens] * n
        samplers = samplers or [None] * n
        logits_processors = logits_processors or [self.logits_processors] * n
        stop_matchers = stop_matchers or [self._default_stop] * n
        return [self._sched.insert(p, m, s or self.sampler, lp or (), sm)
                for p, m, s, lp, sm in zip(prompts, max_tokens, samplers, logits_processors, stop_matchers)]

    def remove(self, uids: Sequence[int], return_prompt_caches: bool = False):
        """Cancel requests at any stage; the next ``next()`` reports each once with ``finish_reason="cancelled"``."""
        self._sched.remove(uids)
        return {} if return_prompt_caches else None

    def next(self) -> Tuple[List[PromptProgress], List[Response]]:
        tic = time.perf_counter()
        prompts, gens = self._sched.next()
        dt = time.perf_counter() - tic
        n_prompt, n_all = self._sched.last_step_prompt_tokens, self._sched.last_step_tokens
        if n_all:   # a step's time is shared between prompt and generation by its tokens
            self._prompt_time += dt * n_prompt / n_all
        self._prompt_tokens += n_prompt
        self._gen_tokens += len(gens)
        if self._sampler.return_logprobs and gens:
            for i, r in enumerate(gens):
                r.logprobs = self._sampler.last_logprobs[i].clone()
        return prompts, gens

    def next_generated(self) -> List[Response]:
        while True:
            prompts, gens = self.next()
            if not gens and prompts:
                continue
            return gens

    @property
    def scheduler(self) -> Scheduler:
        return self._sched


def batch_generate(model, tokenizer, prompts: List[List[int]], prompt_caches=None,
                   max_tokens: Union[int, List[int]] = 128, verbose: bool = False,
                   return_prompt_caches: bool = False, return_token_ids: bool = False,
                   return_logprobs: bool = False, **kwargs) -> BatchResponse:
    """Responses for a batch of token-id prompts (mlx_lm/generate.py:1971-2060).  A token that ends
    a request by a stop sequence is not part of its output."""
    if prompt_caches is not None or return_prompt_caches:
        raise ValueError("prompt caches cannot be passed in or handed out")
    stop = [[t] for t in tokenizer.eos_token_ids] if tokenizer is not None else []
    gen = BatchGenerator(model, stop_tokens=stop, **kwargs)
    n = len(prompts)
    if isinstance(max_tokens, int):
        max_tokens = [max_tokens] * n
    uids = gen.insert(prompts, max_tokens)
    results: Dict[int, List[int]] = {u: [] for u in uids}
    lps: Dict[int, List[float]] = {u: [] for u in uids}
    fin = 0
    with gen.stats() as stats:
        while gen._sched.has_work():
            for r in gen.next_generated():
                if r.finish_reason is not None and verbose:
                    fin += 1
                    print(f"[batch_generate] Finished processing {fin}/{n} ...", end="\r")
                if r.finish_reason not in ("stop", "cancelled"):
                    results[r.uid].append(r.token)
                    lps[r.uid].append(float(r.logprobs))
    gen.close()
    if verbose:
        print(f"[batch_generate] Finished processing {fin}/{n}")
        print(f"[batch_generate] Prompt: {stats.prompt_tokens} tokens, {stats.prompt_tps:.3f} tokens-per-sec")
        print(f"[batch_generate] Generation: {stats.generation_tokens} tokens, "
              f"{stats.generation_tps:.3f} tokens-per-sec")
        print(f"[batch_generate] Peak memory: {stats.peak_memory:.3f} GB")
    texts = [tokenizer.decode(results[u]) if tokenizer is not None else "" for u in uids]
    return BatchResponse(texts, stats, None, [results[u] for u in uids] if return_token_ids else None,
                         [lps[u] for u in uids] if return_logprobs else None)


# ---------------------------------------------------------------------- command line

def str2bool(string: str) -> bool:
    """'F' and 'False' in any case are false, everything else is true (mlx_lm/generate.py:48-49)."""
    return string.lower() not in ["false", "f"]


def setup_arg_parser() -> argparse.ArgumentParser:
    """Options with mlx-lm's names, meanings and defaults (mlx_lm/generate.py:54-213) where this engine has
    the feature; the help texts are this package's own."""
    p = argparse.ArgumentParser(prog="mlx_lm_b200.generate",
                                description="Generate text (or token ids) from a model folder on one GPU")
    p.add_argument("--model", type=str, default=None,
                   help="model folder holding config.json and model*.safetensors")
    p.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                   help="no --model: build a model with random weights drawn from this seed, sized by --config")
    p.add_argument("--config", type=str, default=None, help="the config.json that --random-weights reads")
    p.add_argument("--prompt-tokens", type=str, default=None,
                   help="prompt given as token ids (commas or blanks between them); replaces --prompt")
    p.add_argument("--fp32", action="store_true", help="shorthand for --dtype float32")
    p.add_argument("--extra-eos-token", type=str, default=(), nargs="+",
                   help="further tokens at which generation ends")
    p.add_argument("--prompt", "-p", default=DEFAULT_PROMPT,
                   help="text to continue; '-' takes it from standard input; for a folder without a tokenizer, "
                        "token ids with blanks between them")
    p.add_argument("--max-tokens", "-m", type=int, default=DEFAULT_MAX_TOKENS,
                   help="stop after this many new tokens")
    p.add_argument("--temp", type=float, default=DEFAULT_TEMP, help="temperature; 0 picks the likeliest token")
    p.add_argument("--top-p", type=float, default=DEFAULT_TOP_P,
                   help="nucleus sampling: keep the likeliest tokens whose probabilities add up to this")
    p.add_argument("--min-p", type=float, default=DEFAULT_MIN_P,
                   help="drop tokens less likely than this fraction of the likeliest one")
    p.add_argument("--top-k", type=int, default=DEFAULT_TOP_K, help="keep the k likeliest tokens (0: all)")
    p.add_argument("--xtc-probability", type=float, default=DEFAULT_XTC_PROBABILITY,
                   help="chance, per token, that XTC removes the top choices")
    p.add_argument("--xtc-threshold", type=float, default=DEFAULT_XTC_THRESHOLD,
                   help="XTC removes every candidate above this probability except the least likely of them")
    p.add_argument("--min-tokens-to-keep", type=int, default=DEFAULT_MIN_TOKENS_TO_KEEP,
                   help="candidates that --min-p always leaves")
    p.add_argument("--seed", type=int, default=DEFAULT_SEED,
                   help="seed of the random draws (default: a new one every run)")
    p.add_argument("--ignore-chat-template", action="store_true",
                   help="has no effect: a prompt is always used exactly as given")
    p.add_argument("--verbose", type=str2bool, default=True,
                   help="'T'/'True': also print separators, speeds and memory; 'F'/'False': the response alone")
    p.add_argument("--prefill-step-size", type=int, default=2048, help="prompt tokens run in one step")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16",
                   help="bfloat16: the serving kernels; float32: the whole model in true 32-bit arithmetic")
    p.add_argument("--page-size", type=int, default=16, help="tokens in one page of the key/value cache")
    p.add_argument("--num-pages", type=int, default=None, help="pages in the pool (default: enough for 64 requests)")
    return p


def main(argv: Optional[Sequence[str]] = None) -> None:
    parser = setup_arg_parser()
    args = parser.parse_args(argv)
    if args.fp32:
        args.dtype = "float32"
    if args.prompt_tokens is not None:
        args.prompt = args.prompt_tokens
    tmp = None
    if args.random_weights is not None:
        if args.config is None:
            parser.error("--random-weights needs --config")
        import tempfile

        from .weights import write_random_model
        tmp = tempfile.TemporaryDirectory()
        with open(args.config) as f:
            write_random_model(tmp.name, json.load(f), args.random_weights)
        args.model = tmp.name
    if args.model is None:
        parser.error("--model (or --random-weights with --config) is required")
    model, tokenizer = load(args.model, dtype=args.dtype)
    for t in args.extra_eos_token:
        tokenizer.add_eos_token(t)
    prompt = args.prompt.replace("\\n", "\n").replace("\\t", "\t")
    prompt = sys.stdin.read() if prompt == "-" else prompt
    newline = tokenizer.encode("\n", add_special_tokens=False) if hasattr(tokenizer, "_tokenizer") else []
    sampler = make_sampler(args.temp, args.top_p, args.min_p, args.min_tokens_to_keep, top_k=args.top_k,
                           xtc_probability=args.xtc_probability, xtc_threshold=args.xtc_threshold,
                           xtc_special_tokens=tuple(newline) + tuple(tokenizer.eos_token_ids))
    engine = get_engine(model, page_size=args.page_size, num_pages=args.num_pages, max_requests=1 if args.num_pages
                        else 64)
    response = generate(model, tokenizer, prompt, verbose=args.verbose, max_tokens=args.max_tokens, sampler=sampler,
                        prefill_step_size=args.prefill_step_size, seed=args.seed, engine=engine)
    if not args.verbose:
        print(response)


if __name__ == "__main__":
    main()
