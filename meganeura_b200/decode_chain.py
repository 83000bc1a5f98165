"""The quantized GEMVs of one decode token, column-sharded over the GPUs of a node.

A decode step of a transformer is, per layer, the projections q|k|v, o (+ residual), the
concatenated gate|up projection and the down projection (+ residual), then the lm_head -- the
shapes of meganeura's Qwen3 example (examples/qwen3.rs:243-322) and of its SmolLM2 decode graph
(src/models/smollm2.rs:337-408) after the MatMul+Add and SwiGLU-concat fusions.  This module
runs exactly those dequantize-fused GEMVs, in model order, through the C ABI.

The operators that connect the GEMVs in the model (RMSNorm, RoPE, attention, SwiGLU) are not
part of this library yet, so every GEMV reads a fixed seeded activation vector of the right
length; the exchange steps of the column-sharded model are kept: after q|k|v (a vector of the
attention output's size), after o, after gate|up (the activated half) and after down, the
per-rank output slices are all-gathered so that every rank holds the full vector, and the
lm_head logits are gathered once per token.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import ops, sharding, synth
from ._lib import FMT_Q4, FMT_Q8


@dataclass(frozen=True)
class ModelShape:
    name: str
    layers: int
    hidden: int
    q_dim: int
    kv_dim: int
    ffn: int
    vocab: int


QWEN3_8B = ModelShape("qwen3-8b", 36, 4096, 4096, 1024, 12288, 151936)
SMOLLM2_135M = ModelShape("smollm2-135m", 30, 576, 576, 192, 1536, 49152)


@dataclass(frozen=True)
class GemvSpec:
    name: str          # qkv (or q, k, v), o, gate_up, down, lm_head
    k: int
    n: int
    groups: tuple      # widths of the column groups that are sharded separately (q|k|v, gate|up)
    residual: bool     # fused "+ src" addend (MatMulGemvAdd)
    gather: str        # "" or "first": all-gather this rank's slice of the first column group
    src: str           # which activation vector it reads: "h" (hidden) or "f" (ffn)


def layer_specs(s: ModelShape, fuse_qkv: bool = True) -> list[GemvSpec]:
    """The quantized GEMVs of one layer, in launch order.

    q, k and v read the same vector, so by default they run as one GEMV over the horizontally
    concatenated weight q|k|v -- the transform the reference applies to gate|up
    (HorizontalConcat derived parameter, src/optimize.rs:776-879; blocks never span columns, so
    the concatenation is byte-identical to the three packed weights side by side).
    """
    if fuse_qkv:
        attn = [GemvSpec("qkv", s.hidden, s.q_dim + 2 * s.kv_dim, (s.q_dim, s.kv_dim, s.kv_dim), False, "first", "h")]
    else:
        attn = [GemvSpec("q", s.hidden, s.q_dim, (s.q_dim,), False, "first", "h"),
                GemvSpec("k", s.hidden, s.kv_dim, (s.kv_dim,), False, "", "h"),
                GemvSpec("v", s.hidden, s.kv_dim, (s.kv_dim,), False, "", "h")]
    return attn + [
        GemvSpec("o", s.q_dim, s.hidden, (s.hidden,), True, "first", "h"),
        GemvSpec("gate_up", s.hidden, 2 * s.ffn, (s.ffn, s.ffn), False, "first", "h"),
        GemvSpec("down", s.ffn, s.hidden, (s.hidden,), True, "first", "f"),
    ]


def head_spec(s: ModelShape) -> GemvSpec:
    return GemvSpec("lm_head", s.hidden, s.vocab, (s.vocab,), False, "first", "h")


def gemv_bytes(fmt: int, m: int, k: int, n: int, residual: bool) -> int:
    """Algorithmic bytes of one GEMV: packed weight + activations in + result out (+ addend)."""
    return ops.packed_bytes(fmt, k, n) + 4 * m * k + 4 * m * n * (2 if residual else 1)


def step_bytes(shape: ModelShape, fmt: int, m: int, world: int, layers: int | None = None) -> int:
    """Algorithmic bytes one rank moves per token (its weight slices and its vectors)."""
    total = 0
    nl = shape.layers if layers is None else layers
    for sp in layer_specs(shape):
        total += nl * gemv_bytes(fmt, m, sp.k, sp.n // world, sp.residual)
    hs = head_spec(shape)
    total += gemv_bytes(fmt, m, hs.k, hs.n // world, False)
    return total


class DecodeGemvChain:
    """Device-resident column shards of every projection + the per-token launch sequence."""

    def __init__(self, shape: ModelShape, fmt: int = FMT_Q4, batch: int = 1, rank: int = 0, world: int = 1,
                 layers: int | None = None, seed: int = 0, device=None, group=None, use_plan: bool | None = None,
                 exchange: str = "peer"):
        import torch
        if fmt not in (FMT_Q4, FMT_Q8):
            raise ValueError("fmt must be Q4 or Q8")
        self.shape, self.fmt, self.m, self.rank, self.world = shape, fmt, batch, rank, world
        self.layers = shape.layers if layers is None else layers
        self.group = group
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.launches_per_step = 0
        self.graph = None
        self.plan = None
        # exchange between ranks: "peer" = slices pushed over NVLink by the GEMV itself (mgq_gemv_exchange),
        # "nccl" = all_gather_into_tensor after each exchanging GEMV
        self.exchange = exchange if (world > 1 or exchange == "peer-self") else "none"
        if self.exchange == "peer-self":       # one rank pushing to itself: exercises the exchange code path on one GPU
            self.exchange = "peer"
        self.peer = None
        self.lookahead = True      # every GEMV asks L2 for its successor's weights (mgq_gemv_lookahead)
        # use_plan=True runs the token as one persistent kernel (mgq_plan_*); the default is one
        # kernel per GEMV chained by programmatic dependent launch, which is currently faster
        self.use_plan = bool(use_plan) and world == 1 and batch == 1
        gen = torch.Generator(device="cpu").manual_seed(1000 + seed)
        # fixed activations (replicated on every rank) and residual slices
        self.x = {"h": torch.randn((batch, shape.hidden), generator=gen).to(self.device),
                  "f": torch.randn((batch, shape.ffn), generator=gen).to(self.device)}
        self.x_host = torch.empty((batch, shape.hidden), dtype=torch.float32).pin_memory() if self.device.type == "cuda" else None
        self.ops_list = []
        specs = layer_specs(shape)
        for layer in range(self.layers):
            for sp in specs:
                self.ops_list.append(self._make_op(sp, seed * 100003 + layer * 16 + len(self.ops_list) % 16))
        self.head = self._make_op(head_spec(shape), seed * 100003 + 999983)
        self.ops_list.append(self.head)
        if self.exchange == "peer":
            if batch != 1:
                raise ValueError("the peer exchange takes batch 1; use exchange='nccl'")
            from .exchange import PeerExchange
            self.peer = PeerExchange([op["gather_cols"] for op in self.ops_list], rank, world, group)
            for i, op in enumerate(self.ops_list):
                if op["gather_cols"]:
                    op["full"] = self.peer.gathered(i)
        self.logits = self.head["full"] if self.head["full"] is not None else self.head["y"]
        self.logits_host = torch.empty_like(self.logits, device="cpu").pin_memory() if self.device.type == "cuda" else None

    def _make_op(self, sp: GemvSpec, seed: int) -> dict:
        import torch
        world, rank = self.world, self.rank
        n_loc = sp.n // world
        parts, widths = [], []
        for g, gw in enumerate(sp.groups):
            # this rank's slice of the group: a seeded base of a few hundred columns, tiled on the device
            per_loc = gw // world
            if gw % world != 0 or per_loc % 4 != 0:
                raise ValueError(f"{sp.name}: group of {gw} columns cannot be split over {world} ranks in multiples of 4")
            reps = 1
            for r in range(max(1, per_loc // 256), 0, -1):
                if per_loc % r == 0 and (per_loc // r) % 4 == 0:
                    reps = r
                    break
            base_cols = per_loc // reps
            base = synth.synth_weights(self.fmt, sp.k, base_cols, seed * 7919 + rank * 131 + g)
            parts.append(synth.tile_columns(self.fmt, torch.from_numpy(base).to(self.device), sp.k, base_cols, reps))
            widths.append(per_loc)
        if len(parts) == 1:
            w = parts[0]
        elif self.fmt == FMT_Q8:
            w = torch.cat(parts)
        else:                                              # Q4: all headers first, then all nibbles
            bpc = sp.k // 32
            w = torch.cat([p[: bpc * wd * 4] for p, wd in zip(parts, widths)] +
                          [p[bpc * wd * 4:] for p, wd in zip(parts, widths)])
        assert w.numel() == ops.packed_bytes(self.fmt, sp.k, n_loc)
        y = torch.zeros((self.m, n_loc), dtype=torch.float32, device=self.device)
        addend = None
        if sp.residual:
            addend = torch.randn((self.m, n_loc), generator=torch.Generator().manual_seed(seed + 17)).to(self.device)
        full = None
        gather_cols = 0
        if (world > 1 or self.exchange == "peer") and sp.gather:
            gather_cols = widths[0]
            full = torch.zeros((world * self.m * gather_cols,), dtype=torch.float32, device=self.device)
        return {"spec": sp, "w": w, "y": y, "addend": addend, "full": full, "gather_cols": gather_cols, "n_loc": n_loc}

    # ---------------------------------------------------------------- execution

    def _build_plan(self):
        # every GEMV consumes (a function of) its predecessor's output in the model, so each op
        # waits for the one before it
        self.plan = ops.Plan([(self.fmt, self.x[op["spec"].src], op["w"], op["addend"], op["y"],
                               op["spec"].k, op["n_loc"], i) for i, op in enumerate(self.ops_list)])

    def _launch_all(self):
        import torch.distributed as dist
        if self.use_plan:
            if self.plan is None:
                self._build_plan()
            self.plan.launch()
            self.launches_per_step = 1
            return 1
        if self.exchange == "peer":
            return self._launch_all_peer()
        count = 0
        for i, op in enumerate(self.ops_list):
            sp = op["spec"]
            if self.lookahead and i + 1 < len(self.ops_list):
                ops.lookahead(self.ops_list[i + 1]["w"])
            ops.matmul(self.fmt, self.x[sp.src], op["w"], sp.k, op["n_loc"], addend=op["addend"], out=op["y"], route="gemv")
            count += (self.m + 1) // 2 if self.m > 1 else 1
            if op["full"] is not None:
                src = op["y"] if op["gather_cols"] == op["n_loc"] else op["y"][:, : op["gather_cols"]]
                if self.m > 1 and op["gather_cols"] != op["n_loc"]:
                    src = src.contiguous()
                dist.all_gather_into_tensor(op["full"], src.reshape(-1), group=self.group)
        self.launches_per_step = count
        return count

    def _launch_all_peer(self):
        """Every GEMV pushes its slice to all ranks; each one waits for the exchange before it."""
        import torch
        stream = torch.cuda.current_stream().cuda_stream
        last_exchange = None
        for i, op in enumerate(self.ops_list):
            sp = op["spec"]
            if self.lookahead and i + 1 < len(self.ops_list):
                ops.lookahead(self.ops_list[i + 1]["w"])
            self.peer.gemv(self.fmt, self.x[sp.src], op["w"], op["addend"], op["y"], sp.k, op["n_loc"], i, last_exchange, stream)
            if op["gather_cols"]:
                last_exchange = i
        self.peer.finish(last_exchange, stream)
        self.launches_per_step = len(self.ops_list) + 1
        return self.launches_per_step

    def capture(self):
        """Capture one token's launches into a CUDA graph (falls back to plain launches)."""
        import torch
        self._launch_all()                       # warm-up outside capture (also sizes kernel attributes)
        torch.cuda.synchronize()
        try:
            g = torch.cuda.CUDAGraph()
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                with torch.cuda.graph(g, stream=stream):
                    self._launch_all()
            self.graph = g
        except Exception as exc:                 # pragma: no cover - depends on the NCCL build
            self.graph = None
            self.capture_error = repr(exc)
            torch.cuda.synchronize()
        return self.graph is not None

    def step(self):
        """One token on the device (inputs already resident)."""
        if self.graph is not None:
            self.graph.replay()
        else:
            self._launch_all()

    def step_host(self, x_host_np: np.ndarray | None = None):
        """One token end to end: host activations in, host logits out (synchronous)."""
        import torch
        if x_host_np is not None:
            self.x_host.copy_(torch.from_numpy(x_host_np).reshape(self.x_host.shape))
        self.x["h"].copy_(self.x_host, non_blocking=True)
        self.step()
        self.logits_host.copy_(self.logits, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self.logits_host

    def h2d_bytes(self) -> int:
        return self.x_host.numel() * 4

    def d2h_bytes(self) -> int:
        return self.logits_host.numel() * 4

    def bytes_per_step(self) -> int:
        return step_bytes(self.shape, self.fmt, self.m, self.world, self.layers)
