"""GPT-2: learned absolute positions, pre-LayerNorm blocks with biases, one
fused query/key/value projection, multi-head causal attention, a gelu_new MLP
and an output head tied to the token embedding — the model of
mlx_lm/models/gpt2.py, described with this package's parts.

Differences from that file, both on purpose: ``n_inner`` (null = 4*n_embd)
and ``activation_function`` of config.json are read (mlx-lm hard-codes
4*n_embd, mlx_lm/models/gpt2.py:76-77), and ``n_ctx`` is optional (mlx-lm
requires it and never reads it, :15).  Weights stay in the HF Conv1D layout
``[in, out]`` in the files, as mlx-lm expects them (:175-190).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..config.base import BaseModelArgs, ConfigError, _positive_int
from ..config.registry import register_architecture
from ..parts.linear import ACTIVATIONS
from ..parts import (MLP, Attention, Init, LayerNorm, LearnedAbsolute, ModelDescription, OutputHead, PreNormBlock,
                     TokenEmbedding)


@dataclass
class ModelArgs(BaseModelArgs):
    model_type: str
    n_embd: int
    n_head: int
    n_layer: int
    n_positions: int
    layer_norm_epsilon: float
    vocab_size: int
    n_ctx: Optional[int] = None
    n_inner: Optional[int] = None
    activation_function: str = "gelu_new"
    num_key_value_heads: Optional[int] = None
    # standard deviations of the random-weights mode (HF's initializer_range; not read by mlx-lm)
    initializer_range: float = 0.02
    # random-weights mode only: spread of the LayerNorm gains around 1 (0 = all ones)
    ln_gain_std: float = 0.0

    def validate(self) -> None:
        for k in ("n_embd", "n_head", "n_layer", "n_positions", "vocab_size"):
            _positive_int(k, getattr(self, k))
        if self.n_inner is not None:
            _positive_int("n_inner", self.n_inner)
        if self.n_embd % self.n_head:
            raise ConfigError(f"n_embd ({self.n_embd}) must be divisible by n_head ({self.n_head})")
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.n_head
        if self.num_key_value_heads != self.n_head:
            # mlx_lm/models/gpt2.py:57-58 always gives keys and values n_head heads
            raise ConfigError(f"num_key_value_heads ({self.num_key_value_heads}) must equal n_head ({self.n_head}) "
                              "for GPT-2: its fused c_attn has 3*n_embd outputs")
        if not isinstance(self.layer_norm_epsilon, (int, float)) or self.layer_norm_epsilon <= 0:
            raise ConfigError(f"layer_norm_epsilon must be a positive number, got {self.layer_norm_epsilon!r}")
        if self.activation_function not in ACTIVATION_NAMES:
            raise ConfigError(f"activation_function {self.activation_function!r} is not one of "
                              f"{sorted(ACTIVATION_NAMES)}")
        if self.n_ctx is None:
            self.n_ctx = self.n_positions

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    @property
    def inner_width(self) -> int:
        return 4 * self.n_embd if self.n_inner is None else self.n_inner


def build(args: ModelArgs) -> ModelDescription:
    D = args.n_embd
    w = Init(0.0, args.initializer_range)
    gain = Init(1.0, args.ln_gain_std)
    wte = TokenEmbedding("wte", args.vocab_size, D, init=w)
    wpe = LearnedAbsolute("wpe", args.n_positions, D, init=w)
    blocks = []
    for i in range(args.n_layer):
        p = f"h.{i}"
        blocks.append(PreNormBlock(
            LayerNorm(f"{p}.ln_1", D, args.layer_norm_epsilon, gain_init=gain, bias_init=w),
            Attention(f"{p}.attn", D, args.n_head, args.head_dim, n_kv_heads=args.num_key_value_heads,
                      bias=True, stored="in_out", init=w, bias_init=w),
            LayerNorm(f"{p}.ln_2", D, args.layer_norm_epsilon, gain_init=gain, bias_init=w),
            MLP(f"{p}.mlp", D, args.inner_width, activation=args.activation_function, bias=True,
                stored="in_out", init=w, bias_init=w)))
    return ModelDescription(
        model_type="gpt2", width=D, vocab_size=args.vocab_size, embedding=wte, position=wpe, blocks=blocks,
        final_norm=LayerNorm("ln_f", D, args.layer_norm_epsilon, gain_init=gain, bias_init=w),
        head=OutputHead(args.vocab_size, D, tied_to=wte),
        # causal-mask buffers of HF checkpoints (mlx_lm/models/gpt2.py:173-174 deletes attn.bias)
        ignored_tensors=(r"h\.\d+\.attn\.bias", r"h\.\d+\.attn\.masked_bias"),
        args=args)


# the activations the feed-forward's kernels know (csrc/activations.cuh), less the identity
ACTIVATION_NAMES = frozenset(n for n in ACTIVATIONS if n not in (None, "none"))

register_architecture("gpt2", ModelArgs, build)
