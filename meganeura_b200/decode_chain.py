"""The quantized GEMVs of one decode token, column-sharded over the GPUs of a node.

A decode step of a transformer is, per layer, the projections q|k|v, o (+ residual), the
concatenated gate|up projection and the down projection (+ residual), then the lm_head -- the
shapes of meganeura's Qwen3 example (examples/qwen3.rs:243-322) and of its SmolLM2 decode graph
(src/models/smollm2.rs:337-408) after the MatMul+Add and SwiGLU-concat fusions.  This module
runs exactly those dequantize-fused GEMVs, in model order, through the C ABI, as a chain of real
data dependencies: every GEMV takes as activations the leading columns of its predecessor's output
(q of q|k|v feeds o, the gate half of gate|up feeds down, ...), so no launch can start before the
one before it has finished, exactly as in the model.  The operators that sit between the GEMVs in
the model are the business of decode_model.py.

Weights are what the benchmark configuration describes for the Qwen3-8B-shaped decode: seeded f32
matrices ~ N(0, 0.02^2) run through the reference's quantizer (mgq_quantize_q4 / q8).  A weight of N
columns is the periodic extension of a seeded base of a few hundred columns (30 GB of f32 is never
materialised); the base depends only on (seed, layer, op, column group), so every world size
computes with the same logical weights and a rank's column slice reproduces the unsharded result
bit for bit.

After each sharded GEMV the ranks' slices of its first column group are all-gathered so that every
rank holds the full vector (q, the o output, the gate half, the down output, the logits):
    plan      one persistent kernel per token and rank; slices are pushed into every peer's vector by
              the kernel itself (mgq_plan_create / mgq_plan_create_linked)
    launches  one kernel per GEMV (mgq_gemv; mgq_gemv_exchange or NCCL all-gather when sharded)
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import ops
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


WEIGHT_STD = 0.02
BASE_COLS = 256


def base_weight(fmt: int, k: int, cols: int, seed: int) -> np.ndarray:
    """Packed bytes of a seeded [k, cols] matrix ~ N(0, 0.02^2) after the reference's quantizer."""
    rng = np.random.Generator(np.random.PCG64(seed))
    w = rng.standard_normal((k, cols), dtype=np.float32) * np.float32(WEIGHT_STD)
    return ops.quantize(fmt, w)


def periodic_columns(fmt: int, base_dev, k: int, base_cols: int, c0: int, c1: int):
    """Columns [c0, c1) of the periodic extension of a packed [k, base_cols] weight (device tensors)."""
    import torch
    bpc = k // 32
    idx = torch.arange(c0, c1, device=base_dev.device) % base_cols
    if fmt == FMT_Q8:
        return base_dev.view(base_cols, bpc * 36).index_select(0, idx).reshape(-1)
    hdr = base_dev[: base_cols * bpc * 4].view(base_cols, bpc * 4).index_select(0, idx).reshape(-1)
    nib = base_dev[base_cols * bpc * 4:].view(base_cols, bpc * 16).index_select(0, idx).reshape(-1)
    return hdr, nib


class DecodeGemvChain:
    """Device-resident column shards of every projection + the per-token launch sequence."""

    def __init__(self, shape: ModelShape, fmt: int = FMT_Q4, batch: int = 1, rank: int = 0, world: int = 1,
                 layers: int | None = None, seed: int = 0, device=None, group=None, mode: str = "plan",
                 exchange: str = "peer"):
        import torch
        if fmt not in (FMT_Q4, FMT_Q8):
            raise ValueError("fmt must be Q4 or Q8")
        if mode not in ("plan", "launches"):
            raise ValueError("mode must be 'plan' or 'launches'")
        self.shape, self.fmt, self.m, self.rank, self.world = shape, fmt, batch, rank, world
        self.layers = shape.layers if layers is None else layers
        self.group = group
        self.seed = seed
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        if batch != 1 and mode == "plan":
            mode = "launches"                   # the persistent kernel takes single rows
        self.mode = mode
        # exchange between ranks: "peer" = slices stored over NVLink by the library's own kernels (inside the GEMV
        # for one row, by an all-gather kernel behind the GEMV for a batch of rows), "nccl" =
        # all_gather_into_tensor after each GEMV (launches mode only)
        self.exchange = exchange if world > 1 else "none"
        if self.exchange == "nccl" and mode == "plan":
            raise ValueError("the persistent kernel exchanges through peer memory; use mode='launches' with NCCL")
        self.launches_per_step = 0
        self.graph = None
        self.plan = None
        self.peer = None
        gen = torch.Generator(device="cpu").manual_seed(1000 + seed)
        self.x0 = torch.randn((batch, shape.hidden), generator=gen).to(self.device)      # the token's input vector
        self.x_host = None
        if self.device.type == "cuda":                     # the host copy of the token vector (what step_host sends in)
            self.x_host = torch.empty((batch, shape.hidden), dtype=torch.float32).pin_memory()
            self.x_host.copy_(self.x0)
        self.ops_list = []
        specs = layer_specs(shape)
        for layer in range(self.layers):
            for j, sp in enumerate(specs):
                self.ops_list.append(self._make_op(sp, seed * 100003 + layer * 16 + j))
        self.head = self._make_op(head_spec(shape), seed * 100003 + 999983)
        self.ops_list.append(self.head)
        if self.exchange == "peer":
            from .exchange import PeerExchange
            self.peer = PeerExchange([self.m * op["gather_cols"] for op in self.ops_list], rank, world, group)
            for i, op in enumerate(self.ops_list):
                if self.m == 1:
                    op["full"] = self.peer.gathered(i)
                elif op["gather_cols"]:                              # a batch: the gathered rows, unpacked by the all-gather kernel
                    op["full"] = torch.zeros((self.m, world * op["gather_cols"]), dtype=torch.float32, device=self.device)
        # what each op reads: the token input, then the gathered first group of the op before it
        for i, op in enumerate(self.ops_list):
            k = op["spec"].k
            if i == 0:
                op["x"] = self.x0
            else:
                prev = self.ops_list[i - 1]
                if world * prev["gather_cols"] != k:
                    raise ValueError(f"op {i} reads {k} activations but its predecessor publishes {world * prev['gather_cols']}")
                if world == 1:
                    op["x"] = prev["y"][:, :k]                      # a view: rows are n_loc apart (batch 1: contiguous)
                    if self.m > 1:
                        op["x_buf"] = torch.zeros((self.m, k), dtype=torch.float32, device=self.device)
                elif self.exchange == "nccl" or self.m > 1:
                    op["x"] = prev["full"]
                else:
                    op["x"] = None                                   # taken from the gathered {value, stamp} vector
        self.logits = self.head["full"] if self.head["full"] is not None else self.head["y"]
        self.logits_host = torch.empty((self.m, shape.vocab), dtype=torch.float32).pin_memory() if self.device.type == "cuda" else None

    def _make_op(self, sp: GemvSpec, seed: int) -> dict:
        import torch
        world, rank = self.world, self.rank
        n_loc = sp.n // world
        hdrs, nibs, q8 = [], [], []
        widths = []
        for g, gw in enumerate(sp.groups):
            per_loc = gw // world
            if gw % world != 0 or per_loc % 4 != 0:
                raise ValueError(f"{sp.name}: group of {gw} columns cannot be split over {world} ranks in multiples of 4")
            base_cols = min(BASE_COLS, gw)
            base = torch.from_numpy(base_weight(self.fmt, sp.k, base_cols, seed * 7919 + g)).to(self.device)
            part = periodic_columns(self.fmt, base, sp.k, base_cols, rank * per_loc, (rank + 1) * per_loc)
            if self.fmt == FMT_Q8:
                q8.append(part)
            else:
                hdrs.append(part[0])
                nibs.append(part[1])
            widths.append(per_loc)
        w = torch.cat(q8) if self.fmt == FMT_Q8 else torch.cat(hdrs + nibs)     # Q4: all headers first, then all nibbles
        assert w.numel() == ops.packed_bytes(self.fmt, sp.k, n_loc)
        y = torch.zeros((self.m, n_loc), dtype=torch.float32, device=self.device)
        addend = None
        if sp.residual:
            full_add = torch.randn((self.m, sp.n), generator=torch.Generator().manual_seed(seed + 17))
            addend = full_add[:, rank * n_loc:(rank + 1) * n_loc].contiguous().to(self.device)
        gather_cols = widths[0] if sp.gather else 0
        full = None
        if world > 1 and gather_cols and self.exchange == "nccl":
            full = torch.zeros((self.m, world * gather_cols), dtype=torch.float32, device=self.device)
        return {"spec": sp, "w": w, "y": y, "addend": addend, "full": full, "gather_cols": gather_cols, "n_loc": n_loc}

    # ---------------------------------------------------------------- execution

    def _build_plan(self):
        if self.world == 1:
            self.plan = ops.Plan([(self.fmt, op["x"], op["w"], op["addend"], op["y"], op["spec"].k, op["n_loc"], i)
                                  for i, op in enumerate(self.ops_list)])
            return
        pe = self.peer
        entries, links = [], []
        for i, op in enumerate(self.ops_list):
            entries.append((self.fmt, op["x"], op["w"], op["addend"], op["y"], op["spec"].k, op["n_loc"], 0))
            links.append((pe.push_ptr(i), pe.vec_ptr(i - 1) if i > 0 else None))
        last = len(self.ops_list) - 1
        self.plan = ops.Plan(entries, links=links, epoch_ptr=pe.epoch_ptr, error_ptr=pe.error_ptr,
                             final=(pe.vec_ptr(last), pe.vec_len(last)), keep=pe)

    def _launch_all(self):
        import torch
        import torch.distributed as dist
        if self.mode == "plan":
            if self.plan is None:
                self._build_plan()
            self.plan.launch()
            self.launches_per_step = 1
            return 1
        if self.exchange == "peer":
            return self._launch_all_peer() if self.m == 1 else self._launch_all_peer_rows()
        count = 0
        for op in self.ops_list:
            sp = op["spec"]
            x = op["x"]
            if "x_buf" in op:                                        # batch > 1 on one GPU: rows of the view are not adjacent
                op["x_buf"].copy_(x)
                x = op["x_buf"]
            ops.matmul(self.fmt, x, op["w"], sp.k, op["n_loc"], addend=op["addend"], out=op["y"], route="gemv")
            count += 1
            if op["full"] is not None:
                g = op["gather_cols"]
                parts = op["y"][:, :g].contiguous()
                gathered = torch.empty((self.world, self.m, g), dtype=torch.float32, device=self.device)
                dist.all_gather_into_tensor(gathered.view(-1), parts.view(-1), group=self.group)
                op["full"].copy_(gathered.permute(1, 0, 2).reshape(self.m, self.world * g))
        self.launches_per_step = count
        return count

    def _launch_all_peer(self):
        """Every GEMV pushes its slice to all ranks; each one takes its activations from the vector before it."""
        import torch
        stream = torch.cuda.current_stream().cuda_stream
        for i, op in enumerate(self.ops_list):
            sp = op["spec"]
            self.peer.gemv(self.fmt, op["x"], op["w"], op["addend"], op["y"], sp.k, op["n_loc"], i, i - 1 if i > 0 else None, stream)
        self.peer.finish(len(self.ops_list) - 1, stream)
        self.launches_per_step = len(self.ops_list) + 1
        return self.launches_per_step

    def _launch_all_peer_rows(self):
        """A batch of rows: the 8-row GEMV kernel on the column shard, then one all-gather kernel over peer memory."""
        import torch
        stream = torch.cuda.current_stream().cuda_stream
        count = 0
        for i, op in enumerate(self.ops_list):
            sp = op["spec"]
            ops.matmul(self.fmt, op["x"], op["w"], sp.k, op["n_loc"], addend=op["addend"], out=op["y"], route="gemv")
            count += 1
            g = op["gather_cols"]
            if g:
                self.peer.all_gather_rows(i, op["y"], self.m, g, op["full"], stream)
                count += 1
        self.peer.finish(None, stream)
        self.launches_per_step = count + 1
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
        self.x0.copy_(self.x_host, non_blocking=True)
        self.step()
        self.logits_host.copy_(self.logits_view(), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self.logits_host

    def logits_view(self):
        """The token's logits [batch, vocab] on this rank (the gathered vector when sharded)."""
        if self.world == 1:
            return self.head["y"]
        return self.logits.view(self.m, self.shape.vocab) if self.logits.dim() == 1 else self.logits

    def check_error(self) -> bool:
        """True when a bounded device-side wait ran out since the last check."""
        import torch
        if self.plan is not None:
            try:
                self.plan.check()
            except Exception:
                return True
        if self.peer is not None and self.peer.error():
            return True
        torch.cuda.synchronize()
        return False

    def h2d_bytes(self) -> int:
        return self.x_host.numel() * 4

    def d2h_bytes(self) -> int:
        return self.logits_host.numel() * 4

    def bytes_per_step(self) -> int:
        return step_bytes(self.shape, self.fmt, self.m, self.world, self.layers)
