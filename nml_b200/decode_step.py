"""One decode step of a GPT-OSS-20B-shaped model on the NVFP4 path (benchmark harness).

The layer follows the reference product graph (products/serve/src/gpt_oss/graph.rs:410-573):
RMSNorm -> ``linear_qkv`` -> RoPE (YaRN) -> KV-cache update -> attention with learned sinks
(sliding window of 128 on even layers) -> ``linear`` o_proj -> residual -> RMSNorm -> dense
bf16 router -> ``routed_clamped_swiglu`` -> residual; the model is ``token_embedding``, 24
such layers, RMSNorm and the NVFP4 vocabulary projection (``linear``, graph.rs:601) with a
greedy pick.  Constants are those the reference pins
(products/serve/src/gpt_oss/config.rs:101-142).

Everything NVFP4 (embedding, Q/K/V, o_proj, experts, head) goes through this library's C ABI.
Attention runs on this library's paged-attention decode kernel (page size 16, learned sinks,
sliding window; ``ops.paged_attention_decode``).  The remaining operators stay on the host
framework, as the reference leaves them on its graph: here they are plain torch calls
(RMSNorm, RoPE, cache write, router matmul, arg-max), stand-ins rather than tuned kernels.
Every sequence owns a random set of physical KV pages.

Several GPUs (one process each): sequences are sharded by batch (data-parallel attention, so
the KV read divides too), experts are sharded with the peer-push schedule of
``expert_parallel.ExpertParallelMoE``, the vocabulary projection is column-sharded with a
per-shard arg-max merged across ranks; the attention-side weights are replicas.

Weights are random (N(0, 0.02) quantized with the recipe); ``checkpoint.NvFp4Checkpoint`` reads
stored records, the harness does not need them.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import expert_parallel as ep
from . import ops, quantize


@dataclass(frozen=True)
class GptOssShape:
    """products/serve/src/gpt_oss/config.rs:101-142."""

    layers: int = 24
    hidden: int = 2880
    intermediate: int = 2880
    query_heads: int = 64
    key_value_heads: int = 8
    head_dim: int = 64
    experts: int = 32
    experts_per_token: int = 4
    vocabulary: int = 201088
    sliding_window: int = 128
    rms_norm_eps: float = 1e-5
    rope_theta: float = 150000.0
    rope_factor: float = 32.0
    rope_beta_fast: float = 32.0
    rope_beta_slow: float = 1.0
    original_context: int = 4096
    page_size: int = 16

    @property
    def query_width(self) -> int:
        return self.query_heads * self.head_dim

    @property
    def key_value_width(self) -> int:
        return self.key_value_heads * self.head_dim

    def weight_bytes_per_step(self, batch: int, prior_tokens: int) -> float:
        """HBM bytes one decode step has to move at least (packed weights that the batch
        touches, KV read, head); the bound the step time is compared with."""
        packed = 0.5625  # payload + block scales per weight
        attention = (self.hidden * (self.query_width + 2 * self.key_value_width) +
                     self.query_width * self.hidden) * packed
        experts = self.experts * 3 * self.intermediate * self.hidden * packed
        kv_full = batch * prior_tokens * self.key_value_width * 2 * 2
        kv_window = batch * min(prior_tokens, self.sliding_window) * self.key_value_width * 2 * 2
        head = self.vocabulary * self.hidden * packed
        return (self.layers * (attention + experts) + self.layers // 2 * (kv_full + kv_window) +
                head)


def yarn_inverse_frequencies(shape: GptOssShape, device) -> tuple[torch.Tensor, float]:
    """YaRN-scaled RoPE frequencies and the attention factor (the standard NTK-by-parts rule:
    interpolate below beta_slow rotations over the original context, keep above beta_fast)."""
    half = shape.head_dim // 2
    exponent = torch.arange(0, half, dtype=torch.float64, device=device) / half
    base_frequency = shape.rope_theta ** exponent
    extrapolated = 1.0 / base_frequency
    interpolated = 1.0 / (shape.rope_factor * base_frequency)

    def correction(rotations: float) -> float:
        return half * math.log(shape.original_context / (rotations * 2 * math.pi)) / \
            math.log(shape.rope_theta)

    low = correction(shape.rope_beta_fast)
    high = correction(shape.rope_beta_slow)
    ramp = ((torch.arange(half, dtype=torch.float64, device=device) - low) /
            max(high - low, 1e-3)).clamp(0, 1)
    mask = 1.0 - ramp
    frequencies = interpolated * (1 - mask) + extrapolated * mask
    attention_factor = 0.1 * math.log(shape.rope_factor) + 1.0
    return frequencies.float(), attention_factor


class DecodeModel:
    """Random-init model state of one rank and the decode step over it."""

    def __init__(self, shape: GptOssShape, batch: int, prior_tokens: int, device, group=None,
                 seed: int = 0, layers: int | None = None):
        self.shape = shape
        self.device = device
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if batch % self.world != 0:
            raise ValueError("the batch must divide evenly over the ranks")
        self.batch_total = batch
        self.batch = batch // self.world
        self.prior = prior_tokens
        self.layer_count = shape.layers if layers is None else layers
        capacity = -(-(prior_tokens + 1) // shape.page_size) * shape.page_size
        self.capacity = capacity
        # the same generator on every rank: replicated weights are identical, shards are cut
        # from identical full tensors
        g = torch.Generator(device=device).manual_seed(1234 + seed)
        dtype = torch.bfloat16

        def normal(size, std=0.02):
            return (torch.randn(size, device=device, generator=g) * std).to(dtype)

        def packed(name, size):
            rows = size[-2]
            if len(size) == 2 and rows > 65536:  # bounded temporaries for the vocabulary table
                dense = torch.empty(size, dtype=dtype, device=device)
                for start in range(0, rows, 32768):
                    stop = min(rows, start + 32768)
                    dense[start:stop] = normal((stop - start, size[1]))
            else:
                dense = normal(size)
            return quantize.quantize_parameter(name, dense)

        h, qw, kvw = shape.hidden, shape.query_width, shape.key_value_width
        self.table = packed("embed_tokens", (shape.vocabulary, h))
        head = packed("lm_head", (shape.vocabulary, h))
        self.head = ep.ShardedUnembedding(head, group=group)
        del head
        self.final_norm = torch.ones(h, dtype=dtype, device=device)
        self.exchange = None
        if self.world > 1:
            self.exchange = ep.PeerExchange(-(-self.batch * shape.experts_per_token // 16) * 16,
                                            h, dtype, device, group)
        self.layers = []
        for index in range(self.layer_count):
            layer = {
                "input_norm": torch.ones(h, dtype=dtype, device=device),
                "post_norm": torch.ones(h, dtype=dtype, device=device),
                "q": packed(f"{index}.q", (qw, h)), "q_bias": normal((qw,)),
                "k": packed(f"{index}.k", (kvw, h)), "k_bias": normal((kvw,)),
                "v": packed(f"{index}.v", (kvw, h)), "v_bias": normal((kvw,)),
                "o": packed(f"{index}.o", (h, qw)), "o_bias": normal((h,)),
                "sinks": normal((shape.query_heads,), 1.0).float(),
                "router": normal((shape.experts, h)), "router_bias": normal((shape.experts,)),
                "sliding": index % 2 == 0,
            }
            gate_up = packed(f"{index}.gate_up", (shape.experts, 2 * shape.intermediate, h))
            down = packed(f"{index}.down", (shape.experts, h, shape.intermediate))
            gate_bias = normal((shape.experts, 2 * shape.intermediate))
            down_bias = normal((shape.experts, h))
            if self.world > 1:
                local = ep.LocalExperts.shard(gate_up, gate_bias, down, down_bias, self.rank,
                                              self.world)
                layer["moe"] = ep.ExpertParallelMoE(local, shape.experts_per_token, group=group,
                                                    schedule="push", exchange=self.exchange)
            else:
                layer["experts"] = (gate_up, gate_bias, down, down_bias)
            del gate_up, down
            # paged KV cache of this rank's sequences, [pages, page_size, kv_heads, head_dim]
            # (crates/nml-ir/src/lib.rs:4717-4719); prior tokens hold random keys and values
            pages = self.batch * capacity // shape.page_size
            layer["key"] = normal((pages, shape.page_size, shape.key_value_heads, shape.head_dim),
                                  1.0)
            layer["value"] = normal((pages, shape.page_size, shape.key_value_heads,
                                     shape.head_dim), 1.0)
            self.layers.append(layer)
        pages_per_sequence = capacity // shape.page_size
        order = torch.randperm(self.batch * pages_per_sequence, device=device, generator=g)
        self.page_table = order.view(self.batch, pages_per_sequence).to(torch.int32).contiguous()
        self.lengths = torch.full((self.batch,), prior_tokens + 1, dtype=torch.int32,
                                  device=device)
        # where the new token's key and value go: (physical page, slot) of position `prior`
        self.write_page = self.page_table[:, prior_tokens // shape.page_size].long()
        self.write_slot = prior_tokens % shape.page_size
        frequencies, self.attention_factor = yarn_inverse_frequencies(shape, device)
        angle = frequencies * float(prior_tokens)  # the step decodes position `prior_tokens`
        self.cos = (angle.cos() * self.attention_factor).to(dtype)
        self.sin = (angle.sin() * self.attention_factor).to(dtype)
        self.tokens = torch.randint(0, shape.vocabulary, (self.batch,), device=device,
                                    generator=g, dtype=torch.int32)

    # ------------------------------------------------------------------ pieces
    def _rope(self, x: torch.Tensor) -> torch.Tensor:
        """x [batch, heads, head_dim]; sequential layout: the two halves rotate together."""
        first, second = x[..., : self.shape.head_dim // 2], x[..., self.shape.head_dim // 2:]
        return torch.cat((first * self.cos - second * self.sin,
                          second * self.cos + first * self.sin), dim=-1)

    def _attention(self, layer, query: torch.Tensor) -> torch.Tensor:
        out = ops.paged_attention_decode(
            query, layer["key"], layer["value"], self.page_table, self.lengths, layer["sinks"],
            sliding_window=self.shape.sliding_window if layer["sliding"] else None)
        return out.view(self.batch, self.shape.query_width)

    def _moe(self, layer, hidden: torch.Tensor) -> torch.Tensor:
        # the router is a dense bf16 linear in the reference (graph.rs:552); routing widens it
        logits = F.linear(hidden, layer["router"], layer["router_bias"]).float()
        if self.world > 1:
            return layer["moe"](hidden, logits)
        gate_up, gate_bias, down, down_bias = layer["experts"]
        return ops.routed_clamped_swiglu(hidden, logits, gate_up, gate_bias, down, down_bias,
                                         self.shape.experts_per_token)

    # ------------------------------------------------------------------ the step
    def step(self) -> torch.Tensor:
        """Decodes one token for every sequence of this rank; returns the next token ids."""
        shape, eps = self.shape, self.shape.rms_norm_eps
        hidden = ops.token_embedding(self.table, self.tokens)
        for layer in self.layers:
            x = F.rms_norm(hidden, (shape.hidden,), layer["input_norm"], eps)
            q, k, v = ops.linear_qkv(x, layer["q"], layer["q_bias"], layer["k"], layer["k_bias"],
                                     layer["v"], layer["v_bias"])
            q = self._rope(q.view(self.batch, shape.query_heads, shape.head_dim))
            k = self._rope(k.view(self.batch, shape.key_value_heads, shape.head_dim))
            layer["key"][self.write_page, self.write_slot] = k
            layer["value"][self.write_page, self.write_slot] = v.view(
                self.batch, shape.key_value_heads, shape.head_dim)
            attention = self._attention(layer, q)
            hidden = ops.linear(attention, layer["o"], layer["o_bias"], residual=hidden)
            x = F.rms_norm(hidden, (shape.hidden,), layer["post_norm"], eps)
            hidden = hidden + self._moe(layer, x)
        x = F.rms_norm(hidden, (shape.hidden,), self.final_norm, eps)
        return self.head.argmax(x)
