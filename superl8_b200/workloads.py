"""Synthetic workloads with the shapes and value distributions of the five benchmark
configurations of this path (all inputs are ~N(0,1) fp16; nothing is read from disk).

cfg1  B1  Hq8  Hkv2 S1024 D128 causal
cfg2  B1  Hq32 Hkv8 S4096 D128 causal
cfg3  B16 Hq64 Hkv8 S8192 D128 causal, a seeded 1 % of the (head, channel) pairs of Q and of K x20
cfg4  B8  Hq16 Hkv1 S2048 D in {64, 256} non-causal (+ ragged lengths in [100, 2048])
cfg5  decode: B128 Hq64 Hkv8 D128, context length per sequence uniform in [1024, 32768]
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class PrefillCfg:
    name: str
    B: int
    Hq: int
    Hkv: int
    S: int
    D: int
    causal: bool
    outliers: bool = False

    @property
    def ops(self) -> float:
        """4 B Hq M N D, halved when causal (the reference's count, bench/harness.py:220-223)."""
        return 4.0 * self.B * self.Hq * self.S * self.S * self.D * (0.5 if self.causal else 1.0)

    @property
    def units(self) -> int:
        """Independent (batch, kv-head) units."""
        return self.B * self.Hkv


PREFILL = {
    "cfg1": PrefillCfg("cfg1", 1, 8, 2, 1024, 128, True),
    "cfg2": PrefillCfg("cfg2", 1, 32, 8, 4096, 128, True),
    "cfg3": PrefillCfg("cfg3", 16, 64, 8, 8192, 128, True, outliers=True),
    "cfg4_d64": PrefillCfg("cfg4_d64", 8, 16, 1, 2048, 64, False),
    "cfg4_d256": PrefillCfg("cfg4_d256", 8, 16, 1, 2048, 256, False),
}


def outlier_channels(H: int, D: int, seed: int, frac: float = 0.01) -> torch.Tensor:
    """Boolean [H, D]: the ceil(frac H D) (head, channel) pairs that are scaled x20."""
    n = math.ceil(frac * H * D)
    idx = torch.randperm(H * D, generator=torch.Generator().manual_seed(seed))[:n]
    mask = torch.zeros(H * D, dtype=torch.bool)
    mask[idx] = True
    return mask.view(H, D)


def _cfg_index(cfg: PrefillCfg) -> int:
    """Seed base of a configuration: the first digit of its name ("cfg3" -> 3), 0 for a name without one."""
    digits = "".join(ch for ch in cfg.name if ch.isdigit())
    return int(digits[:1]) if digits else 0


def _apply_outliers(cfg: PrefillCfg, q, k):
    """x20 on the seeded 1 % of (head, channel) pairs of q [..., Hq, S, D] and k [..., Hkv, S, D] (in place)."""
    qm = outlier_channels(cfg.Hq, cfg.D, 7).to(q.device)
    km = outlier_channels(cfg.Hkv, cfg.D, 8).to(k.device)
    q.mul_(torch.where(qm, 20.0, 1.0).to(q.dtype).view(cfg.Hq, 1, cfg.D))
    k.mul_(torch.where(km, 20.0, 1.0).to(k.dtype).view(cfg.Hkv, 1, cfg.D))


def prefill_element_cpu(cfg: PrefillCfg, b: int, outliers: bool | None = None, dtype=torch.float16):
    """Batch element ``b`` of a configuration on the CPU, reproducible anywhere: Q [Hq,S,D], then K, then V
    [Hkv,S,D] drawn in that order from ``torch.Generator().manual_seed(1000 * cfg + b)``, ~N(0,1), cast to
    ``dtype``; the outlier channels of cfg3 are applied after the cast.  A (batch, kv-head) unit is the slice
    q[g*h:g*(h+1)], k[h:h+1], v[h:h+1] with g = Hq / Hkv."""
    g = torch.Generator().manual_seed(1000 * _cfg_index(cfg) + b)
    q = torch.randn(cfg.Hq, cfg.S, cfg.D, generator=g).to(dtype)
    k = torch.randn(cfg.Hkv, cfg.S, cfg.D, generator=g).to(dtype)
    v = torch.randn(cfg.Hkv, cfg.S, cfg.D, generator=g).to(dtype)
    if cfg.outliers if outliers is None else outliers:
        _apply_outliers(cfg, q, k)
    return q, k, v


def prefill_inputs(cfg: PrefillCfg, device, first_unit_batch: int = 0, outliers: bool | None = None,
                   source: str = "device"):
    """fp16 Q [B,Hq,S,D], K, V [B,Hkv,S,D] on ``device``.  ``source="device"`` draws from the device
    generator seeded by (configuration, first batch index) -- fast, what the benchmark times;
    ``source="cpu"`` stacks prefill_element_cpu(cfg, first_unit_batch + i), the per-element CPU seeds a
    checker can re-create without the device."""
    if source == "cpu":
        els = [prefill_element_cpu(cfg, first_unit_batch + i, outliers) for i in range(cfg.B)]
        return tuple(torch.stack([e[j] for e in els]).to(device) for j in range(3))
    g = torch.Generator(device=device)
    g.manual_seed(1000 * _cfg_index(cfg) + first_unit_batch)
    q = torch.randn(cfg.B, cfg.Hq, cfg.S, cfg.D, device=device, dtype=torch.float16, generator=g)
    k = torch.randn(cfg.B, cfg.Hkv, cfg.S, cfg.D, device=device, dtype=torch.float16, generator=g)
    v = torch.randn(cfg.B, cfg.Hkv, cfg.S, cfg.D, device=device, dtype=torch.float16, generator=g)
    if cfg.outliers if outliers is None else outliers:
        _apply_outliers(cfg, q, k)
    return q, k, v


def ragged_lengths(cfg: PrefillCfg, lo: int = 100) -> torch.Tensor:
    """Per-sequence lengths of the ragged arm of cfg4: uniform in [lo, S] from seed 4004 (int32 [B])."""
    g = torch.Generator().manual_seed(4004)
    return torch.randint(lo, cfg.S + 1, (cfg.B,), generator=g, dtype=torch.int32)


@dataclass(frozen=True)
class DecodeCfg:
    name: str = "cfg5"
    B: int = 128
    Hq: int = 64
    Hkv: int = 8
    D: int = 128
    n_min: int = 1024
    n_max: int = 32768


def decode_lengths(cfg: DecodeCfg, first_seq: int = 0, count: int | None = None) -> torch.Tensor:
    """Context length of every sequence of the GLOBAL batch (seeded), then this shard's slice."""
    count = cfg.B if count is None else count
    g = torch.Generator().manual_seed(5005)
    total = max(first_seq + count, cfg.B)
    lens = torch.randint(cfg.n_min, cfg.n_max + 1, (total,), generator=g, dtype=torch.int32)
    return lens[first_seq:first_seq + count].contiguous()


def decode_bytes(lens: torch.Tensor, Hkv: int, D: int) -> float:
    """Algorithmic bytes of one decode step: int8 K + fp32 scale + fp16 V per key and KV head."""
    return float(lens.sum().item()) * Hkv * (D + 4 + 2 * D)


def decode_inputs(cfg: DecodeCfg, lens: torch.Tensor, device):
    """q fp16 [B,Hq,1,D]; K cache int8 [B,Hkv,Nmax,D] + fp32 scales [B,Hkv,Nmax] made by quantising
    ~N(0,1) fp16 keys with this library's K prologue (per-sequence statistics); V cache fp16."""
    from . import quant
    B = lens.numel()
    n_max = int(lens.max().item())
    g = torch.Generator(device=device)
    g.manual_seed(5000)
    q = torch.randn(B, cfg.Hq, 1, cfg.D, device=device, dtype=torch.float16, generator=g)
    v = torch.randn(B, cfg.Hkv, n_max, cfg.D, device=device, dtype=torch.float16, generator=g)
    k_i8 = torch.empty(B, cfg.Hkv, n_max, cfg.D, device=device, dtype=torch.int8)
    k_scale = torch.empty(B, cfg.Hkv, n_max, device=device, dtype=torch.float32)
    ldev = lens.to(device)
    step = 16
    for b0 in range(0, B, step):
        k = torch.randn(min(step, B - b0), cfg.Hkv, n_max, cfg.D, device=device, dtype=torch.float16, generator=g)
        mean = quant.k_mean(k, ldev[b0:b0 + step].contiguous())
        ki, ks, _ = quant.smooth_quantize_k(k, mean)
        k_i8[b0:b0 + step] = ki
        k_scale[b0:b0 + step] = ks.squeeze(-1)
    return q, k_i8, k_scale, v, ldev
