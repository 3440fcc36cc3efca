"""Tensor-parallel quantized linear layers of a LLaMA decoder block (host side).

Mirrors how the reference's FasterTransformer fork shards the four linear layers of a block
(LlamaDecoderLayerWeight.cc:378-400; TensorParallelGptContextAttentionLayer.cc:50-53,
TensorParallelSiluFfnLayer.cc:53-57):

* QKV, gate, up: **column parallel** -- every rank owns a slice of the output features (rows of every weight plane),
  no communication;
* O, down: **row parallel** -- every rank owns a slice of the input features (word columns of every weight plane),
  produces a full ``[M, hidden]`` fp16 partial, and the partials are summed by an all-reduce.

Bit-planes shard cleanly both ways; slices along K are whole 128-feature units (the pack / MMA granularity), dealt as
evenly as possible (11008 = 86 units -> 22/22/21/21 for four ranks).  Activations are quantised with a static scale
(the reference's quantiser, mode 0), so ranks need not agree on a per-token scale for row-parallel inputs; partial
sums are reduced after dequantisation, in fp16, as FasterTransformer does.

The arithmetic is injected (``backend``): the product backend is :class:`AbqBackend` (this library, CUDA only);
tests drive the sharding logic with a numpy stand-in over ``gloo`` ranks.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple


def unit_ranges(total: int, parts: int, unit: int = 128) -> List[Tuple[int, int]]:
    """[begin, end) of every part when ``total`` features are dealt in whole ``unit``-feature pieces, the first
    ``total/unit % parts`` parts getting one piece more."""
    if total % unit:
        raise ValueError(f"{total} is not a multiple of {unit}")
    units = total // unit
    base, extra = divmod(units, parts)
    out, at = [], 0
    for r in range(parts):
        n = (base + (1 if r < extra else 0)) * unit
        out.append((at, at + n))
        at += n
    return out


@dataclass
class LinearSpec:
    name: str
    out_features: int
    in_features: int
    parallel: str  # "column" (split out_features) or "row" (split in_features, all-reduce after)


def llama_block_specs(hidden: int, ffn: int) -> List[LinearSpec]:
    """The four quantized GEMMs of a block as FasterTransformer runs them: fused QKV, O, fused gate+up, down."""
    return [LinearSpec("qkv", 3 * hidden, hidden, "column"), LinearSpec("o", hidden, hidden, "row"),
            LinearSpec("gate_up", 2 * ffn, hidden, "column"), LinearSpec("down", hidden, ffn, "row")]


def shard_of(spec: LinearSpec, rank: int, world: int, unit: int = 128) -> Tuple[slice, slice]:
    """(rows, columns) of the full [out_features][in_features] code matrix that ``rank`` owns."""
    if spec.parallel == "column":
        # fused layers (qkv, gate_up) are split per fused part so that every rank holds matching slices of each
        parts = 3 if spec.name == "qkv" else (2 if spec.name == "gate_up" else 1)
        per = spec.out_features // parts
        b, e = unit_ranges(per, world, unit)[rank]  # the same ranges as the K split of the row-parallel layer that follows
        rows = [i for p in range(parts) for i in range(p * per + b, p * per + e)]
        return rows, slice(0, spec.in_features)
    b, e = unit_ranges(spec.in_features, world, unit)[rank]
    return slice(0, spec.out_features), slice(b, e)


class TensorParallelBlockLinears:
    """The linear layers of one decoder block on one rank.

    ``backend.make_linear(codes, scale, zero, w_bits, group, reduce_output=...)`` returns an object with
    ``__call__(x_half) -> fp16``; ``backend.all_reduce(t)`` returns the sum over ranks (in ``t`` or in a tensor of its own); ``backend.glue`` supplies the elementwise stand-ins between the
    GEMMs (attention itself is outside this path: the first third of the QKV output stands in for its result).
    """

    def __init__(self, backend, hidden: int, ffn: int, rank: int, world: int, weights: Sequence, w_bits: int, group: int = 0):
        self.backend, self.hidden, self.ffn, self.rank, self.world = backend, hidden, ffn, rank, world
        self.specs = llama_block_specs(hidden, ffn)
        self.layers = {}
        for spec, (codes, scale, zero) in zip(self.specs, weights):
            rows, cols = shard_of(spec, rank, world)
            c = codes[rows][:, cols]
            if group:  # per-group parameters follow their K groups
                gsl = slice(cols.start // group, cols.stop // group)
                s, z = scale[rows][:, gsl], (None if zero is None else zero[rows][:, gsl])
            else:      # per-channel parameters follow the rows (replicated for row-parallel layers)
                s, z = scale[rows], (None if zero is None else zero[rows])
            self.layers[spec.name] = backend.make_linear(c, s, z, w_bits, group, reduce_output=spec.parallel == "row")

    def _buf(self, name, M):
        # where a layer exposes the buffer its plan reads, the producing elementwise step writes straight into it
        return self.layers[name].input(M) if hasattr(self.layers[name], "input") else None

    # The block in the three pieces that lie between its two all-reduces (a caller that replays CUDA graphs captures
    # the pieces and launches the collectives between them):
    def attention_part(self, x):
        """x -> this rank's partial of the attention output projection (to be all-reduced)."""
        be, M = self.backend, x.shape[0]
        qkv = self.layers["qkv"](x)                                                        # [M][3 * hidden / world]
        attn = be.glue_attention(qkv, self.layers["qkv"].out_features // 3, self._buf("o", M))  # this rank's heads
        return self.layers["o"](attn)                                                      # partial [M][hidden]

    def ffn_part(self, x, o):
        """(x, all-reduced o) -> (h, this rank's partial of the down projection (to be all-reduced))."""
        be, M = self.backend, x.shape[0]
        h = be.glue_residual(x, o, self._buf("gate_up", M))
        gu = self.layers["gate_up"](h)                                                     # [M][2 * ffn_local]
        act = be.glue_swiglu(gu, self.layers["gate_up"].out_features // 2, self._buf("down", M))
        return h, self.layers["down"](act)                                                 # partial [M][hidden]

    def input_buffer(self, M):
        """Where this block's first layer reads its activations: a caller that chains blocks hands it to the block before
        as ``out_to`` (None with backends that keep no such buffers)."""
        return self._buf("qkv", M)

    def forward(self, x, out_to=None):
        """x: fp16 [M][hidden], replicated on every rank.  Returns fp16 [M][hidden], replicated (in ``out_to`` if given)."""
        be = self.backend
        if getattr(be, "fuses_residual", False):
            return self._forward_fused_residual(x, out_to)
        o = be.all_reduce(self.attention_part(x))
        h, d = self.ffn_part(x, o)
        return be.glue_residual(h, be.all_reduce(d), out_to)

    def _forward_fused_residual(self, x, out_to=None):
        """The same block with both residual adds done where the row-parallel layer's sum is finished (the GEMM's epilogue,
        or the all-reduce kernel behind it): h = x + O(attn) lands in the gate/up layer's input buffer, the block's
        output is h + down(act).  Same arithmetic as forward(): the fp16 sum rounded, then an fp16 add."""
        be, M = self.backend, x.shape[0]
        qkv = self.layers["qkv"](x)
        attn = be.glue_attention(qkv, self.layers["qkv"].out_features // 3, self._buf("o", M))
        h = be.linear_sum_plus(self.layers["o"], attn, x, self._buf("gate_up", M), "h")
        gu = self.layers["gate_up"](h)
        act = be.glue_swiglu(gu, self.layers["gate_up"].out_features // 2, self._buf("down", M))
        return be.linear_sum_plus(self.layers["down"], act, h, out_to, "y")


class AbqLinear:
    """One sharded quantized linear layer on the GPU: one GEMM call that quantises the fp16 activations with a static
    scale (ABQ_FLAG_X_HALF) and writes fp16 through its fused dequantisation (per-channel or per-group scale and zero
    point, per-token activation scale).  The weights are re-ordered once at construction into the decode kernel's
    prepared form (ABQ_FLAG_WEIGHTS_PREPARED); a row-parallel layer on several ranks can have the sum over the ranks
    done inside the GEMM (``fused_reduce``: abq_fused_allreduce over symmetric memory)."""

    def __init__(self, abq, torch, codes, scale, zero, w_bits: int, group: int, x_bits: int = 8, x_scale: float = 16.0,
                 max_tokens: int = 64, make_out=None, fused_reduce=None, status=None, fused_rows: int = 1 << 30):
        self.abq, self.torch = abq, torch
        self.make_out = make_out  # row-parallel layers: output buffers that the other ranks can read
        self.out_features, self.in_features = codes.shape
        N, K = codes.shape
        self.w_bits, self.x_bits, self.group = w_bits, x_bits, group
        self.planes = torch.empty((w_bits, N, K // 32), dtype=torch.int32, device="cuda")
        abq.pack_int32(codes.to(torch.int32).contiguous(), self.planes, N, K, w_bits)
        self.scale = scale.to(torch.float16).contiguous()
        self.zero = None if zero is None else zero.to(torch.uint8).contiguous()
        self.q_scale = torch.full((1,), x_scale, dtype=torch.float32, device="cuda")
        self.max_tokens = max_tokens
        self.inv = torch.full((max_tokens,), 1.0 / x_scale, dtype=torch.float32, device="cuda")
        self.work = torch.empty(max(256, abq.gemm_workspace_bytes(max_tokens, N, K, x_bits, w_bits)), dtype=torch.uint8, device="cuda")
        self.status = status
        self.plans = {}
        self.inputs = {}
        self.needs_reduce = False  # set by the backend: a row-parallel layer on several ranks
        self.prepared = None
        self.prepared_done = False
        self.fused = None
        self.fused_rows = fused_rows  # token counts up to this use the fused sum (where there is one), larger ones make_out
        self.on_fused_output = None   # told the output buffer of every plan whose GEMM already delivers the sum
        if fused_reduce is not None:  # (dist, world, rank): receive buffers + flags of all ranks in one symmetric allocation
            import torch.distributed._symmetric_memory as symm
            dist, world, rank = fused_reduce
            tiles = (N + 15) // 16
            recv_bytes = 2 * world * max_tokens * N * 2
            flag_bytes = 2 * world * tiles * 4
            buf = symm.empty(((recv_bytes + 255) // 256 * 256 + flag_bytes,), dtype=torch.uint8, device="cuda")
            buf.zero_()
            h = symm.rendezvous(buf, dist.group.WORLD)
            torch.cuda.synchronize()
            dist.barrier()  # every rank's flags are zero before anybody's first GEMM
            base = [int(p) for p in h.buffer_ptrs]
            counter = torch.zeros(2, dtype=torch.int32, device="cuda")
            self.fused = dict(buf=buf, handle=h, counter=counter,
                              desc=abq.make_fused_allreduce(world, rank, base, [b + (recv_bytes + 255) // 256 * 256 for b in base], counter, max_tokens))

    def _plan(self, M, residual=None, out_to=None):
        """Plan and output buffer per token count, made on first use (outside stream capture: planning may touch the
        workspace) and reused afterwards, so that a captured graph replays launches only.  ``residual`` (fp16 [M][N]) is
        added to the result by the GEMM itself; ``out_to`` makes the GEMM write into a caller's buffer (the next layer's
        input) -- both only where this rank's GEMM delivers the final value (no separate all-reduce behind it)."""
        key = (M, None if residual is None else residual.data_ptr(), None if out_to is None else out_to.data_ptr())
        if key not in self.plans:
            B = self.abq.binding
            fused = self.fused if M <= self.fused_rows else None
            if out_to is not None:
                out = out_to
            else:
                out = (self.make_out(M, self.out_features) if (self.make_out and fused is None) else
                       self.torch.empty((M, self.out_features), dtype=self.torch.float16, device="cuda"))
            x_view = self.input(M)  # the GEMM reads fp16 here (one buffer per token count, whatever the plan)
            flags = self.abq.FLAG_PDL | self.abq.FLAG_X_HALF
            kw = dict(x_bits=self.x_bits, w_bits=self.w_bits, x_signed=True, w_signed=False, out_dtype=self.abq.OUT_FP16,
                      scale_mode=self.abq.SCALE_GROUP if self.group else self.abq.SCALE_CHANNEL, group_size=self.group,
                      w_scale=self.scale, w_zero=self.zero, x_scale=self.inv, x_quant_scale=self.q_scale, workspace=self.work,
                      status_word=self.status, residual=residual)
            probe = B.make_params(M, self.out_features, self.in_features, x_view, self.planes, out, flags=flags, **kw)
            nbytes = self.abq.gemm_prepared_weight_bytes(probe) if M <= 32 else 0
            st = None
            if nbytes:
                if self.prepared is None:
                    self.prepared = self.torch.empty(nbytes, dtype=self.torch.uint8, device="cuda")
                try:
                    st = self.abq.gemm_init(B.make_params(M, self.out_features, self.in_features, x_view, self.planes, out,
                                                          flags=flags | self.abq.FLAG_WEIGHTS_PREPARED, route=self.abq.ROUTE_I8_MMA,
                                                          w_prepared=self.prepared, allreduce=None if fused is None else fused["desc"], **kw))
                except self.abq.AbqError:
                    st = None
                    if fused is not None:
                        raise
                if st is not None and not self.prepared_done:
                    self.abq.gemm_prepare_weights(st)
                    self.torch.cuda.synchronize()  # a PDL GEMM must not be launched behind the kernel that writes its weights
                    self.prepared_done = True
            if st is None:
                if fused is not None:
                    raise RuntimeError("the fused all-reduce needs the prepared-weights decode kernel")
                st = self.abq.gemm_init(probe)
            if fused is not None and self.on_fused_output is not None:
                self.on_fused_output(out)
            self.plans[key] = (st, x_view, out)
        return self.plans[key]

    def input(self, M):
        """The fp16 buffer [M][in_features] this layer's plan reads: producers write straight into it."""
        if M not in self.inputs:
            self.inputs[M] = self.torch.empty((M, self.in_features), dtype=self.torch.float16, device="cuda")
        return self.inputs[M]

    def sums_in_gemm(self, M):
        """True where this layer's GEMM call delivers the finished value: one rank, or the all-reduce fused into its epilogue."""
        return not self.needs_reduce or (self.fused is not None and M <= self.fused_rows)

    def __call__(self, x, residual=None, out_to=None):
        M = x.shape[0]
        if M > self.max_tokens:
            raise ValueError(f"{M} tokens, planned for at most {self.max_tokens}")
        st, x_view, out = self._plan(M, residual, out_to)
        if x.data_ptr() != x_view.data_ptr():
            x_view.copy_(x)  # callers that cannot write into input(M) pay one copy; the GEMM call quantises x_view itself
        self.abq.gemm_exec(st)
        return out


class AbqBackend:
    """Product backend: this library for the GEMMs, torch.distributed (NCCL) for the all-reduce, torch elementwise
    kernels for the glue between the GEMMs."""

    def __init__(self, abq, torch, dist=None, x_bits: int = 8, x_scale: float = 16.0, max_tokens: int = 64):
        if not torch.cuda.is_available():
            raise RuntimeError("AbqBackend needs a CUDA device: there is no CPU path")
        self.abq, self.torch, self.dist = abq, torch, dist
        self.x_bits, self.x_scale, self.max_tokens = x_bits, x_scale, max_tokens
        import os
        several = dist is not None and dist.get_world_size() > 1
        # how the row-parallel partials are summed: "peer" (the library's one-shot all-reduce kernel after the GEMM), "fused"
        # (inside the GEMM's epilogue), "nccl" (torch.distributed), or "auto" (default) = whichever of the first two measured
        # faster on 2, 4 and 8 ranks: fused for up to 8 tokens (no launch of its own, one flag round trip instead of two),
        # peer above (the fused form ties the layer to the prepared-weights kernel, and for the tensor-parallel shapes at
        # 9..16 rows per launch the plane-reading kernel is the faster one)
        self.reduce_kind = os.environ.get("ABQ_TP_REDUCE", "nccl" if os.environ.get("ABQ_TP_NCCL", "0") == "1" else "auto") if several else "none"
        if self.reduce_kind not in ("none", "auto", "fused", "peer", "nccl"):
            raise ValueError(f"ABQ_TP_REDUCE={self.reduce_kind}")
        self.fused_rows = {"fused": 1 << 30, "auto": 8 if several else 0}.get(self.reduce_kind, 0)
        if self.reduce_kind == "auto" and "ABQ_TP_FUSED_ROWS" in os.environ:
            self.fused_rows = int(os.environ["ABQ_TP_FUSED_ROWS"])
        self.peer_reduce = self.reduce_kind in ("auto", "fused", "peer")  # no NCCL call on the data path: the step can be one CUDA graph
        self._reduced = {}
        self._fused_outputs = set()
        self.status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def make_linear(self, codes, scale, zero, w_bits, group, reduce_output=False):
        make_out = self._peer_visible_output if (reduce_output and self.reduce_kind in ("auto", "peer")) else None
        fused = (self.dist, self.dist.get_world_size(), self.dist.get_rank()) if (reduce_output and self.fused_rows > 0) else None
        layer = AbqLinear(self.abq, self.torch, codes, scale, zero, w_bits, group, self.x_bits, self.x_scale, self.max_tokens, make_out,
                          fused_reduce=fused, status=self.status, fused_rows=self.fused_rows)
        layer.needs_reduce = bool(reduce_output and self.dist is not None and self.dist.get_world_size() > 1)
        # all_reduce() leaves the outputs of fused plans alone: the GEMM already summed them
        layer.on_fused_output = lambda out: self._fused_outputs.add(out.data_ptr())
        return layer

    # ---- all-reduce of the row-parallel partials.  Several ranks on one node: the partial buffers live in symmetric
    # memory (every rank has every rank's buffer mapped) and the library's one-shot kernel adds them over NVLink peer
    # loads -- one launch, capturable in a CUDA graph.  Otherwise (or with ABQ_TP_NCCL=1): torch.distributed.
    def _peer_visible_output(self, M, N):
        import torch.distributed._symmetric_memory as symm
        t = symm.empty((M, N), dtype=self.torch.float16, device="cuda")
        h = symm.rendezvous(t, self.dist.group.WORLD)
        self._reduced[t.data_ptr()] = (h, t, self.torch.empty((M, N), dtype=self.torch.float16, device="cuda"),
                                       self.torch.zeros(2, dtype=self.torch.int32, device="cuda"))
        return t

    fuses_residual = True  # TensorParallelBlockLinears may call linear_sum_plus()

    def linear_sum_plus(self, layer, x_in, residual, out_to, tag):
        """residual + (sum over the ranks of layer(x_in)), written to ``out_to`` where given: inside the GEMM where its call
        delivers the finished value, inside the peer all-reduce kernel behind it otherwise; with NCCL (or more than 32
        tokens, where the tensor-core route has no residual input) as separate steps."""
        M = x_in.shape[0]
        if M <= 32 and layer.sums_in_gemm(M):
            return layer(x_in, residual=residual, out_to=out_to)
        part = layer(x_in)
        entry = self._reduced.get(part.data_ptr()) if M <= 32 else None
        if entry is None:
            return self.glue_residual(residual, self.all_reduce(part), out_to)
        h, _, own_out, counter = entry
        out = own_out if out_to is None else out_to
        self.abq.peer_allreduce_half(h.buffer_ptrs_dev, h.signal_pad_ptrs_dev, h.rank, h.world_size, h.signal_pad_size // 8, out, part.numel(),
                                     counter, self.status, residual=residual)
        return out

    def all_reduce(self, t):
        if self.dist is None or self.dist.get_world_size() == 1 or t.data_ptr() in self._fused_outputs:
            return t
        entry = self._reduced.get(t.data_ptr())
        if entry is None:
            self.dist.all_reduce(t)
            return t
        h, _, out, counter = entry
        # the upper half of the pad: the lower words belong to the symmetric-memory library's own barriers
        self.abq.peer_allreduce_half(h.buffer_ptrs_dev, h.signal_pad_ptrs_dev, h.rank, h.world_size, h.signal_pad_size // 8, out, t.numel(),
                                     counter, self.status)
        return out

    def glue_attention(self, qkv, hl, out=None):
        if out is None:
            return qkv[:, :hl].contiguous()
        out.copy_(qkv[:, :hl])
        return out

    def glue_residual(self, a, b, out=None):
        if out is None:
            out = self.torch.empty_like(a)
        if a.numel() % 8 == 0 and a.is_contiguous() and b.is_contiguous():
            self.abq.add_half(a, b, out, a.numel())   # one launch, chained to the GEMMs around it
            return out
        return self.torch.add(a, b, out=out)

    def glue_swiglu(self, gu, fl, out=None):
        if out is None:
            out = self.torch.empty((gu.shape[0], fl), dtype=gu.dtype, device=gu.device)
        if fl % 8 == 0 and gu.is_contiguous() and gu.shape[1] == 2 * fl:
            self.abq.swiglu_half(gu, out, gu.shape[0], fl)
            return out
        return self.torch.mul(self.torch.nn.functional.silu(gu[:, :fl]), gu[:, fl:], out=out)
