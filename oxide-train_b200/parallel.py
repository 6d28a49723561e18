"""The three places the GEMM path shards across the GPUs of one box.

The reference is single-GPU (SPEC.md:15); these are new.  One process per GPU,
``torch.distributed`` (NCCL over NVLink / NVSwitch) for the exchange steps, the
kernels of this package for the compute.  Each class keeps its exchange logic
in plain tensor code that also runs on CPU tensors over the ``gloo`` backend;
the compute is reached through a small ``ops`` object so that tests can stand
in a CPU implementation for it.

* :class:`VocabParallelHead` — fused lm-head + cross-entropy with the vocabulary
  split over ranks; one all-gather of the per-row statistics and one merge
  kernel in the forward, the sum of ``d_hidden`` over the shards in the
  backward (copy-engine reduce-scatter under the weight-gradient GEMM, or
  NCCL's all-reduce).
* :class:`ExpertParallelMoe` — experts split over ranks, tokens split over
  ranks; on GPUs the exchange is driven from the device (counts gathered by
  the barrier kernel, rows dispatched into and fetched from peer memory by
  this library's kernels, token slices as a pipeline); over ``gloo`` a counts
  exchange and two all-to-alls.
* :class:`TensorParallelMlp` — column-parallel up, row-parallel down,
  reduce-scatter of the partial outputs, in row pieces so that the exchange of
  one piece overlaps the GEMMs of the next.
* :class:`PeerRowExchange`, :class:`PeerBarrier` — what the above share on
  GPUs: row blocks moved by the copy engines between peer-mapped buffers, and
  a one-block barrier kernel over peer memory.

On GPUs the classes keep their large buffers between steps: what ``forward`` /
``backward`` return is valid until the next call of the same method.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

TILE_N = 256


# --------------------------------------------------------------------------- compute back end

class DeviceOps:
    """The package's kernels, as the parallel classes call them."""

    def __init__(self, gemm):
        from . import moe as _moe
        from .lmhead import FusedLmHead
        self.gemm = gemm
        self._moe = _moe
        self._FusedLmHead = FusedLmHead

    # lm-head shard
    def head_forward_shard(self, hidden, weight_shard, local_targets, classes_local, w_layout):
        import ctypes as C
        from . import _lib as L
        from .gemm import _stream_ptr
        m, k = hidden.shape
        v_local = weight_shard.shape[1] if w_layout == "in_out" else weight_shard.shape[0]
        dev = hidden.device
        need = self.gemm._lib.b200gemm_lmhead_ce_workspace_bytes(m)
        if getattr(self, "_ws", None) is None or self._ws.numel() < need:
            self._ws = torch.empty(need, dtype=torch.uint8, device=dev)
        # one [3, m] block (row_max, row_sum, row_target_logit): what the ranks all-gather
        out = torch.empty((3, m), dtype=torch.float32, device=dev)
        L.check(self.gemm._lib.b200gemm_lmhead_ce_forward_shard(
            self.gemm._h, _stream_ptr(), hidden.data_ptr(), weight_shard.data_ptr(),
            L.MN_MAJOR if w_layout == "in_out" else L.K_MAJOR, local_targets.data_ptr(), m, k, v_local,
            classes_local, out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(),
            self._ws.data_ptr(), self._ws.numel()))
        return out

    def head_merge_shards(self, gathered):
        """``gathered`` is ``[world, 3, m]``: returns ``(lse, row_loss, loss)`` from one launch."""
        from . import _lib as L
        from .gemm import _stream_ptr
        world, _, m = gathered.shape
        dev = gathered.device
        lse = torch.empty(m, dtype=torch.float32, device=dev)
        row_loss = torch.empty(m, dtype=torch.float32, device=dev)
        loss = torch.empty(1, dtype=torch.float32, device=dev)
        L.check(self.gemm._lib.b200gemm_lmhead_ce_merge_shards(
            self.gemm._h, _stream_ptr(), gathered.data_ptr(), world, m, lse.data_ptr(), row_loss.data_ptr(),
            loss.data_ptr()))
        return lse, row_loss, loss

    def head_backward_shard(self, hidden, weight_shard, local_targets, lse, classes_local, w_layout, dy,
                            d_weight, accumulate_dw):
        head = self._FusedLmHead(self.gemm, classes_local, w_layout)
        return head.backward(hidden, weight_shard, local_targets, lse, dy=dy, d_weight=d_weight,
                             accumulate_dw=accumulate_dw)

    def head_dlogits(self, hidden, weight_shard, local_targets, lse, classes_local, w_layout, dy, out=None):
        """First step of the shard's backward: the logits recomputed into bf16 dlogits."""
        head = self._FusedLmHead(self.gemm, classes_local, w_layout)
        dl, _, _ = head.backward(hidden, weight_shard, local_targets, lse, dy=dy, dlogits=out,
                                 want_d_hidden=False, want_d_weight=False)
        return dl

    def head_dhidden_partial(self, dlogits, weight_shard, w_layout, dtype, out=None):
        """This shard's part of d_hidden = dlogits . W_shard^T, in `dtype`."""
        k = weight_shard.shape[0] if w_layout == "in_out" else weight_shard.shape[1]
        dh = torch.empty((dlogits.shape[0], k), dtype=dtype, device=dlogits.device) if out is None else out
        self.gemm.gemm(dlogits, weight_shard, dh, transposed_b=(w_layout != "in_out"))
        return dh

    def widen(self, t, out=None):
        return self.gemm.convert_bf16_to_f32(t, out)

    def head_dweight(self, hidden, dlogits, w_layout, d_weight, accumulate_dw):
        """Second half: d_weight (=|+=) hidden^T . dlogits in the weight's orientation."""
        k, v = hidden.shape[1], dlogits.shape[1]
        if d_weight is None:
            shape = (k, v) if w_layout == "in_out" else (v, k)
            d_weight = torch.zeros(shape, dtype=torch.float32, device=hidden.device)
            accumulate_dw = True
        a, b = (hidden, dlogits) if w_layout == "in_out" else (dlogits, hidden)
        self.gemm.gemm(a, b, d_weight, transposed_a=True, transposed_b=True, accumulate=accumulate_dw)
        return d_weight

    # MoE
    def route(self, scores, top_k, scores_are_logits):
        return self._moe.route(self.gemm, scores, top_k, scores_are_logits=scores_are_logits)

    def scatter(self, x, routing):
        return self._moe.scatter(self.gemm, x, routing)

    def combine(self, y_permuted, routing, residual, out_dtype):
        return self._moe.combine(self.gemm, y_permuted, routing, residual, out_dtype)

    def combine_into(self, y_permuted, routing, residual, out):
        from . import _lib as L
        from .gemm import _stream_ptr
        L.check(self.gemm._lib.b200gemm_moe_combine(
            self.gemm._h, _stream_ptr(), y_permuted.data_ptr(), routing.dest_row.data_ptr(),
            routing.gate_weights.data_ptr(), residual.data_ptr() if residual is not None else None,
            routing.tokens, routing.top_k, y_permuted.shape[1], out.data_ptr(),
            L.OUT_F32 if out.dtype == torch.float32 else L.OUT_BF16))
        return out

    def grouped_indexed(self, a, b, offsets, group_b_index, silu):
        from . import _lib as L
        from .gemm import _stream_ptr
        rows, k = a.shape
        n = b.shape[2]                                  # b is [experts_local, k, n]
        out = torch.empty((rows, n), dtype=torch.bfloat16, device=a.device)
        if rows == 0:
            return out
        L.check(self.gemm._lib.b200gemm_grouped_gemm_indexed(
            self.gemm._h, _stream_ptr(), a.data_ptr(), a.stride(0), b.data_ptr(), L.MN_MAJOR,
            b.stride(1), b.stride(0), b.shape[0], group_b_index.data_ptr(), out.data_ptr(),
            out.stride(0), offsets.data_ptr(), group_b_index.numel(), rows, n, k, int(silu)))
        return out

    def grouped_indexed_into(self, a, b, offsets, group_b_index, silu, out):
        from . import _lib as L
        from .gemm import _stream_ptr
        rows, k = a.shape
        n = b.shape[2]
        L.check(self.gemm._lib.b200gemm_grouped_gemm_indexed(
            self.gemm._h, _stream_ptr(), a.data_ptr(), a.stride(0), b.data_ptr(), L.MN_MAJOR,
            b.stride(1), b.stride(0), b.shape[0], group_b_index.data_ptr(), out.data_ptr(),
            out.stride(0), offsets.data_ptr(), group_b_index.numel(), rows, n, k, int(silu)))
        return out

    def ep_plan(self, all_counts, world, rank, experts):
        from . import _lib as L
        from .gemm import _stream_ptr
        dev = all_counts.device
        dst_base = torch.empty(experts, dtype=torch.int32, device=dev)
        offsets = torch.empty(experts + 1, dtype=torch.int32, device=dev)
        index = torch.empty(experts, dtype=torch.int32, device=dev)
        L.check(self.gemm._lib.b200gemm_moe_ep_plan(self.gemm._h, _stream_ptr(), all_counts.data_ptr(), world,
                                                    rank, experts, dst_base.data_ptr(), offsets.data_ptr(),
                                                    index.data_ptr()))
        return dst_base, offsets, index

    def ep_return_plan(self, all_counts, world, rank, experts):
        from . import _lib as L
        from .gemm import _stream_ptr
        dev = all_counts.device
        dst_rank = torch.empty(experts, dtype=torch.int32, device=dev)
        dst_row = torch.empty(experts, dtype=torch.int32, device=dev)
        L.check(self.gemm._lib.b200gemm_moe_ep_return_plan(self.gemm._h, _stream_ptr(), all_counts.data_ptr(), world,
                                                           rank, experts, dst_rank.data_ptr(), dst_row.data_ptr()))
        return dst_rank, dst_row

    def grouped_indexed_peer(self, a, b, offsets, group_b_index, peer_ptrs, world, ld_out, out_rows, dst_rank, dst_row):
        """The expert GEMM whose epilogue stores each (source rank, expert) group's rows into that
        rank's buffer (``peer_ptrs``: every rank's buffer as seen from here)."""
        from . import _lib as L
        from .gemm import _stream_ptr
        rows, k = a.shape
        n = b.shape[2]
        L.check(self.gemm._lib.b200gemm_grouped_gemm_peer(
            self.gemm._h, _stream_ptr(), a.data_ptr(), a.stride(0), b.data_ptr(), L.MN_MAJOR, b.stride(1),
            b.stride(0), b.shape[0], group_b_index.data_ptr(), peer_ptrs, world, ld_out, out_rows,
            dst_rank.data_ptr(), dst_row.data_ptr(), offsets.data_ptr(), group_b_index.numel(), rows, n, k))

    def ep_push(self, x, routing, dst_base, peer_ptrs, inbox_rows, world, experts):
        from . import _lib as L
        from .gemm import _stream_ptr
        tokens, d = x.shape
        L.check(self.gemm._lib.b200gemm_moe_ep_push(
            self.gemm._h, _stream_ptr(), x.data_ptr(), routing.selected_experts.data_ptr(),
            routing.slots.data_ptr(), dst_base.data_ptr(), peer_ptrs, inbox_rows, world, experts, tokens,
            routing.top_k, d))

    def ep_pull_combine(self, peer_ptrs, routing, dst_base, residual, result_rows, world, experts, d, out):
        from . import _lib as L
        from .gemm import _stream_ptr
        L.check(self.gemm._lib.b200gemm_moe_ep_pull_combine(
            self.gemm._h, _stream_ptr(), peer_ptrs, routing.selected_experts.data_ptr(),
            routing.slots.data_ptr(), dst_base.data_ptr(), routing.gate_weights.data_ptr(),
            residual.data_ptr() if residual is not None else None, result_rows, world, experts,
            routing.tokens, routing.top_k, d, out.data_ptr(),
            L.OUT_F32 if out.dtype == torch.float32 else L.OUT_BF16))
        return out

    # dense GEMMs (weights are [IN, OUT], read in place)
    def linear(self, x, w, out_dtype=torch.bfloat16, out=None):
        y = torch.empty((x.shape[0], w.shape[1]), dtype=out_dtype, device=x.device) if out is None else out
        self.gemm.gemm(x, w, y, transposed_b=True)
        return y

    def linear_input_grad(self, dy, w, out_dtype=torch.bfloat16, out=None):
        dx = torch.empty((dy.shape[0], w.shape[0]), dtype=out_dtype, device=dy.device) if out is None else out
        self.gemm.gemm(dy, w, dx)
        return dx

    def linear_input_grad_into(self, dy, w, dx):
        self.gemm.gemm(dy, w, dx)

    def linear_weight_grad(self, x, dy, dw):
        self.gemm.f32_accumulate_transposed(x, dy, dw)

    def peer_barrier(self, peer_words, world, rank, epoch, limit_ms, payload=None, peer_tables=None):
        """Launches the barrier kernel on the current stream (``peer_words`` / ``peer_tables``:
        ctypes arrays of every rank's buffer as seen from here)."""
        from . import _lib as L
        from .gemm import _stream_ptr
        L.check(self.gemm._lib.b200gemm_peer_barrier(
            self.gemm._h, _stream_ptr(), peer_words, world, rank, epoch, limit_ms,
            payload.data_ptr() if payload is not None else None,
            payload.numel() if payload is not None else 0, peer_tables))

    def sum_parts(self, parts, out):
        """``out = sum_p parts[p]`` (``parts`` is ``[p, ...]``, contiguous), added in fp32 in order."""
        from . import _lib as L
        from .gemm import _stream_ptr
        code = lambda t: L.OUT_F32 if t.dtype == torch.float32 else L.OUT_BF16
        L.check(self.gemm._lib.b200gemm_sum_parts(
            self.gemm._h, _stream_ptr(), parts.data_ptr(), code(parts), parts.stride(0), parts.shape[0],
            out.numel(), out.data_ptr(), code(out), 0))
        return out


def _world(group):
    return dist.get_world_size(group), dist.get_rank(group)


def nccl_group_with_cta_limit(max_ctas: int, ranks=None):
    """A second NCCL process group over the same ranks whose collectives use at most
    ``max_ctas`` thread blocks (one SM each): the partner of ``reserve_sms`` below -- the GEMMs
    leave that many SMs free and the collective is told to fit into them."""
    opts = dist.ProcessGroupNCCL.Options()
    opts.config.max_ctas = int(max_ctas)
    opts.config.min_ctas = 1
    ranks = list(range(dist.get_world_size())) if ranks is None else list(ranks)
    return dist.new_group(ranks=ranks, pg_options=opts)


class _ReservedSms:
    """``with _ReservedSms(ops, n):`` -- GEMMs launched inside spread over all but ``n`` SMs.

    A persistent GEMM CTA takes all of an SM's shared memory, so a collective's kernel that
    becomes ready while a GEMM runs waits for whole GEMM CTAs to finish -- and a GEMM that
    starts while the collective holds some SMs runs part of its statically scheduled
    clusters as a second wave.  Keeping ``n`` SMs out of the GEMM grid (the collective is
    given a channel limit to match) lets both run side by side."""

    def __init__(self, ops, sms: int):
        self.gemm = getattr(ops, "gemm", None) if sms else None
        self.sms = sms

    def __enter__(self):
        if self.gemm is not None:
            total = torch.cuda.get_device_properties(self.gemm.device).multi_processor_count
            self.before = self.gemm.sm_limit            # a limit the caller set outlives this block
            in_force = self.before or total
            self.gemm.set_sm_limit(max(2, min(in_force, total - self.sms)))
        return self

    def __exit__(self, *exc):
        if self.gemm is not None:
            self.gemm.set_sm_limit(self.before)
        return False


# --------------------------------------------------------------------------- vocabulary-parallel head

def vocab_shards(vocab_padded: int, world: int, tile: int = TILE_N):
    """Column ranges ``[(c0, c1), ...]`` per rank: whole 256-column tiles, as even as they come.

    50432 columns are 197 tiles; over 8 ranks that is 25, 25, 25, 25, 25, 24, 24, 24."""
    tiles = (vocab_padded + tile - 1) // tile
    base, rem = divmod(tiles, world)
    out, c = [], 0
    for r in range(world):
        n = (base + (1 if r < rem else 0)) * tile
        out.append((min(c, vocab_padded), min(c + n, vocab_padded)))
        c += n
    return out


def merge_softmax_stats(row_max, row_sum, row_target_logit, group=None):
    """All-reduce the shards' per-row statistics into ``(lse, row_loss, mean_loss)``.

    One MAX all-reduce of ``row_max`` and one SUM all-reduce of the rescaled sums
    stacked with the target logits (2 x rows floats)."""
    gmax = row_max.clone()
    dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
    packed = torch.stack([row_sum * torch.exp(row_max - gmax), row_target_logit])
    dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
    lse = gmax + torch.log(packed[0])
    row_loss = lse - packed[1]
    return lse, row_loss, row_loss.double().mean().float()


class VocabParallelHead:
    def __init__(self, ops, classes: int, vocab_padded: int, group=None, w_layout: str = "in_out",
                 reduce_dtype=torch.bfloat16, reserve_sms: int = 0, exchange: str = "nccl",
                 d_hidden: str = "all", barrier: str = "kernel"):
        self.ops, self.group, self.w_layout, self.reduce_dtype = ops, group, w_layout, reduce_dtype
        self.barrier = barrier              # how the copy exchange orders the ranks (PeerRowExchange)
        self.reserve_sms = reserve_sms      # SMs the weight-gradient GEMM leaves to d_hidden's exchange
        # d_hidden's sum over the shards: "nccl" = all_reduce; "copy" = copy-engine reduce-scatter
        # (+ all-gather) through peer memory, see PeerRowExchange.  d_hidden = "all": every rank
        # gets all rows; "scatter": rank r gets rows [r * m / world, (r + 1) * m / world) only --
        # half the bytes, and what a row-parallel layer below the head wants anyway.
        self.exchange, self.d_hidden, self._px, self._px_key = exchange, d_hidden, None, None
        self.world, self.rank = _world(group)
        self.c0, self.c1 = vocab_shards(vocab_padded, self.world)[self.rank]
        self.classes_local = max(0, min(classes, self.c1) - self.c0)
        self._side = None
        self._lt = None
        self._keep = None                   # buffers of the backward, kept between steps

    def shard_weight(self, weight_full):
        """This rank's columns of a full ``[hidden, vocab_padded]`` weight (a copy)."""
        if self.w_layout == "in_out":
            return weight_full[:, self.c0:self.c1].contiguous()
        return weight_full[self.c0:self.c1].contiguous()

    def local_targets(self, targets):
        """Targets relative to this shard's first column; kept from the forward for the backward
        of the same batch."""
        cached = self._lt
        if cached is not None and cached[0] is targets and cached[1] == targets._version:
            return cached[2]
        lt = (targets - self.c0).to(torch.int32)
        self._lt = (targets, targets._version, lt)
        return lt

    def forward(self, hidden, weight_shard, targets):
        lt = self.local_targets(targets)
        stats = self.ops.head_forward_shard(hidden, weight_shard, lt, self.classes_local, self.w_layout)
        if hasattr(self.ops, "head_merge_shards") and hidden.device.type == "cuda":
            # ONE collective (an all-gather of every rank's [3, rows] block, 384 KB per rank at
            # 32768 rows) and ONE kernel, instead of a MAX all-reduce, a SUM all-reduce and the
            # elementwise passes between them.
            gathered = torch.empty((self.world,) + tuple(stats.shape), dtype=stats.dtype, device=stats.device)
            dist.all_gather_into_tensor(gathered, stats, group=self.group)
            lse, row_loss, loss = self.ops.head_merge_shards(gathered)
        else:
            lse, row_loss, loss = merge_softmax_stats(*stats, group=self.group)
        return loss, lse, row_loss

    def backward(self, hidden, weight_shard, targets, lse, dy: float = 1.0, d_weight=None,
                 accumulate_dw: bool = False):
        """Returns ``(dlogits shard, d_hidden summed over shards, d_weight shard)``.  On CUDA the
        first two are buffers of this object: valid until the next ``backward``."""
        lt = self.local_targets(targets)
        if not hasattr(self.ops, "head_dweight") or hidden.device.type != "cuda":
            dl, dh, dw = self.ops.head_backward_shard(hidden, weight_shard, lt, lse, self.classes_local,
                                                      self.w_layout, dy, d_weight, accumulate_dw)
            dist.all_reduce(dh, op=dist.ReduceOp.SUM, group=self.group)
            return dl, dh, dw
        # d_hidden's all-reduce (rows x hidden, the one large message of this path) runs on
        # a side stream underneath the weight-gradient GEMM.  The shards' partial sums
        # travel as bf16 -- the reference's own d_hidden is a bf16 GEMM output that is
        # widened afterwards (gpu/model/src/lib.rs:3125-3145, 5777-5784) -- which halves
        # the message; `reduce_dtype=torch.float32` keeps fp32 partials instead.
        # The large intermediates (dlogits: rows x local vocabulary; the d_hidden partial; this
        # rank's rows of the sum; the widened result) live in buffers this object keeps: a step
        # in steady state allocates nothing, and what is returned is valid until the next call.
        m, k = hidden.shape
        v_local = weight_shard.shape[1] if self.w_layout == "in_out" else weight_shard.shape[0]
        key = (m, k, v_local, self.reduce_dtype, hidden.device)
        if self._keep is None or self._keep["key"] != key:
            dev, share = hidden.device, (m // self.world if m % self.world == 0 else m)
            self._keep = {"key": key,
                          "dl": torch.empty((m, v_local), dtype=torch.bfloat16, device=dev),
                          "dh": torch.empty((m, k), dtype=self.reduce_dtype, device=dev),
                          "mine": torch.empty((share, k), dtype=self.reduce_dtype, device=dev),
                          "wide": {}}
        keep = self._keep
        dl = self.ops.head_dlogits(hidden, weight_shard, lt, lse, self.classes_local, self.w_layout, dy,
                                   out=keep["dl"])
        dh = self.ops.head_dhidden_partial(dl, weight_shard, self.w_layout, self.reduce_dtype, out=keep["dh"])
        if self._side is None:
            self._side = torch.cuda.Stream(device=hidden.device)
        self._side.wait_stream(torch.cuda.current_stream())
        use_copy = self.exchange == "copy" and self.world > 1 and m % self.world == 0
        scatter = self.d_hidden == "scatter" and m % self.world == 0
        if use_copy and (self._px is None or self._px_key != (m, k, dh.dtype)):
            self._px = PeerRowExchange(self.ops, self.group, dh.device, [m // self.world], k, dh.dtype,
                                       barrier=self.barrier)
            self._px_key = (m, k, dh.dtype)
        mine = keep["mine"] if (use_copy or scatter) else None
        with torch.cuda.stream(self._side):
            if use_copy:
                self._px.reduce_scatter(0, dh, mine)
                summed = mine if scatter else self._px.all_gather(0, mine)
            elif scatter:
                dist.reduce_scatter_tensor(mine, dh, op=dist.ReduceOp.SUM, group=self.group)
                summed = mine
            else:
                dist.all_reduce(dh, op=dist.ReduceOp.SUM, group=self.group)
                summed = dh
        dh = summed
        with _ReservedSms(self.ops, self.reserve_sms):
            dw = self.ops.head_dweight(hidden, dl, self.w_layout, d_weight, accumulate_dw)
        torch.cuda.current_stream().wait_stream(self._side)
        if dh.dtype != torch.float32:
            wide = keep["wide"].get(tuple(dh.shape))
            if wide is None:
                wide = keep["wide"][tuple(dh.shape)] = torch.empty(dh.shape, dtype=torch.float32, device=dh.device)
            dh = self.ops.widen(dh, wide)
        return dl, dh, dw


# --------------------------------------------------------------------------- expert-parallel MoE

def exchange_counts(counts_by_expert, world, group=None):
    """``counts_by_expert`` [experts] (rows this rank routes to every expert) ->
    ``(send_counts [world, local], recv_counts [world, local])``; ``recv_counts[s, e]`` is
    the number of rows rank ``s`` sends to this rank's local expert ``e``."""
    local = counts_by_expert.numel() // world
    send = counts_by_expert.reshape(world, local).to(torch.int64).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return send, recv


def received_groups(recv_counts):
    """Groups of the received rows, one per (source rank, local expert), in arrival order:
    ``(offsets int32 [groups + 1], group_b_index int32 [groups])``."""
    world, local = recv_counts.shape
    flat = recv_counts.reshape(-1)
    offsets = torch.zeros(flat.numel() + 1, dtype=torch.int32, device=flat.device)
    offsets[1:] = torch.cumsum(flat, 0).to(torch.int32)
    index = torch.arange(local, dtype=torch.int32, device=flat.device).repeat(world)
    return offsets, index


class ExpertParallelMoe:
    """``y = combine(down(silu(up(dispatch(x)))))`` with experts and tokens split over ranks.

    ``w_up_local`` is ``[experts / world, d, ff]``, ``w_down_local`` ``[experts / world, ff, d]``."""

    def __init__(self, ops, experts: int, top_k: int, w_up_local, w_down_local, group=None, pieces=1,
                 use_peer_copies: bool = False, exchange: str = "nccl", return_path: str = "pull",
                 barrier: str = "kernel", exchange_ctas: int = 48, exchange_bulk: bool = True):
        self.ops, self.group, self.experts, self.top_k = ops, group, experts, top_k
        # device exchange: thread blocks of the dispatch / combine kernels that run beside an
        # expert GEMM (0 = two per SM) and whether they are the bulk-copy forms, which fill the
        # links from the few SMs `reserve_sms` keeps free of GEMM CTAs.  The first slice's
        # dispatch and the last slice's combine have the GPU to themselves and always spread
        # over all of it.
        self.exchange_ctas, self.exchange_bulk = exchange_ctas, exchange_bulk
        # device exchange, how the ranks wait for one another: "kernel" = this library's barrier
        # kernel, which also gathers the per-expert counts (PeerBarrier); "nccl" = an all-gather
        # of the counts and one-element all-reduces
        self.barrier = barrier
        self.pieces, self._side = pieces, None
        self.use_peer_copies, self._peer, self._peer_shape, self._index = use_peer_copies, None, None, None
        self.exchange, self._dev = exchange, None       # "nccl" | "device" (peer stores / loads)
        # device exchange, how results come back: "pull" = the token's rank reads each result row
        # from its owner (peer loads) while it combines; "push" = the owner's down-projection GEMM
        # stores its rows into the token rank's buffer from its epilogue, and the combine is local
        self.return_path = return_path
        self.reserve_sms = 24                           # SMs kept free of GEMM CTAs in the device path
        self.world, self.rank = _world(group)
        if experts % self.world:
            raise ValueError("experts must divide evenly over the ranks")
        self.w_up, self.w_down = w_up_local, w_down_local
        self.last = {}

    def forward(self, x, scores, scores_are_logits=False, residual=None, out_dtype=torch.float32):
        if self.world == 1:
            # one rank owns every expert: the routed rows are already where they are multiplied
            r = self.ops.route(scores, self.top_k, scores_are_logits)
            xp = self.ops.scatter(x, r)                   # rows sorted by expert
            index = torch.arange(self.experts, dtype=torch.int32, device=x.device)
            hidden = self.ops.grouped_indexed(xp, self.w_up, r.offsets, index, True)
            yp = self.ops.grouped_indexed(hidden, self.w_down, r.offsets, index, False)
            self.last = {"rows_received": xp.shape[0], "rows_sent": xp.shape[0], "routing": r}
            return self.ops.combine(yp, r, residual, out_dtype)
        if self.exchange == "device" and x.device.type == "cuda":
            return self._forward_device(x, scores, scores_are_logits, residual, out_dtype)
        if self.use_peer_copies and x.device.type == "cuda":
            return self._forward_peer(x, scores, scores_are_logits, residual, out_dtype)
        return self._forward_pipelined(x, scores, scores_are_logits, residual, out_dtype)

    def _forward_device(self, x, scores, scores_are_logits, residual, out_dtype):
        """Several GPUs, device-driven exchange: nothing is read back to the host.

        Per slice of tokens: route; gather the per-expert counts (on the barrier kernel's
        way, or NCCL's all-gather); a plan kernel turns them into inbox offsets; a dispatch
        kernel puts every routed row straight into its expert owner's inbox (peer memory);
        barrier; the two grouped GEMMs run on what arrived; barrier; a combine kernel
        fetches each result row from its owner's result buffer.  The slices form a pipeline
        (see ``_forward_device_body``), so the NVLink traffic of one slice runs beside the
        tensor-core work of its neighbours; the whole step is enqueued without a host
        round trip."""
        import ctypes as C
        n, d = x.shape
        ff, d_out = self.w_up.shape[2], self.w_down.shape[2]
        slices = self._slices(n)
        caps = [rows * self.top_k * self.world for _, rows in slices]   # worst case: every row of every rank lands here
        first = [sum(caps[:i]) for i in range(len(caps))]               # first buffer row of every slice
        total = sum(caps)
        key = (tuple(slices), d, ff, d_out)
        if self._dev is None or self._dev["key"] != key:
            import torch.distributed._symmetric_memory as symm_mem
            grp = self.group if self.group is not None else dist.group.WORLD
            inbox = symm_mem.empty((total, d), dtype=torch.bfloat16, device=x.device)
            results = symm_mem.empty((total, d_out), dtype=torch.bfloat16, device=x.device)
            h_in = symm_mem.rendezvous(inbox, grp.group_name)
            h_res = symm_mem.rendezvous(results, grp.group_name)
            ptrs_in, ptrs_res = [], []
            for p in range(len(slices)):
                a_in = (C.c_void_p * self.world)()
                a_res = (C.c_void_p * self.world)()
                for r in range(self.world):
                    a_in[r] = h_in.get_buffer(r, (total, d), torch.bfloat16).data_ptr() + first[p] * d * 2
                    a_res[r] = h_res.get_buffer(r, (total, d_out), torch.bfloat16).data_ptr() + first[p] * d_out * 2
                ptrs_in.append(a_in)
                ptrs_res.append(a_res)
            pair_rows = [rows * self.top_k for _, rows in slices]
            pair_first = [sum(pair_rows[:i]) for i in range(len(pair_rows))]
            returned = symm_mem.empty((sum(pair_rows), d_out), dtype=torch.bfloat16, device=x.device)
            h_back = symm_mem.rendezvous(returned, grp.group_name)
            ptrs_back = []
            for p in range(len(slices)):
                a_back = (C.c_void_p * self.world)()
                for r in range(self.world):
                    a_back[r] = (h_back.get_buffer(r, (sum(pair_rows), d_out), torch.bfloat16).data_ptr()
                                 + pair_first[p] * d_out * 2)
                ptrs_back.append(a_back)
            self._dev = {"key": key, "inbox": inbox, "results": results, "handles": (h_in, h_res, h_back),
                         "ptrs_in": ptrs_in, "ptrs_res": ptrs_res, "returned": returned, "ptrs_back": ptrs_back,
                         "pair_rows": pair_rows, "pair_first": pair_first,
                         "hidden": torch.empty((total, ff), dtype=torch.bfloat16, device=x.device),
                         "token": torch.zeros(1, device=x.device),
                         # one barrier object per slice: each slice's kernels stay on one stream
                         "barriers": ([PeerBarrier(self.ops, grp, x.device, payload_count=self.experts)
                                       for _ in slices] if self.barrier == "kernel" else None)}
        dv = self._dev
        # the result lives in a buffer this object keeps (valid until the next forward): a step
        # in steady state allocates nothing large, so the caching allocator never grows while
        # the host runs ahead of the GPU
        out = dv.get(("out", out_dtype))
        if out is None:
            out = dv[("out", out_dtype)] = torch.empty((n, d_out), dtype=out_dtype, device=x.device)
        # The expert GEMMs leave `reserve_sms` SMs to the neighbouring slices' dispatch and
        # combine kernels (and to NCCL's barriers, where those are used).
        with _ReservedSms(self.ops, self.reserve_sms):
            return self._forward_device_body(x, scores, scores_are_logits, residual, out, dv, slices, caps, first)

    def _slices(self, n):
        """``[(first token, tokens), ...]``: ``pieces`` equal slices, or -- ``pieces`` a list of
        weights -- slices in those proportions (a short first and last slice shorten what no GEMM
        can cover: the first slice's dispatch and the last slice's combine)."""
        if isinstance(self.pieces, int):
            pieces = self.pieces if (n % self.pieces == 0 and n // self.pieces >= 256) else 1
            return [(p * (n // pieces), n // pieces) for p in range(pieces)]
        total = sum(self.pieces)
        rows = [n * w // total for w in self.pieces]
        if sum(rows) != n or min(rows) < 256:
            return [(0, n)]
        return [(sum(rows[:i]), rows[i]) for i in range(len(rows))]

    def _forward_device_body(self, x, scores, scores_are_logits, residual, out, dv, slices, caps, first):
        n = x.shape[0]
        d_out = out.shape[1]
        pieces = len(slices)
        # With the barrier kernel every slice has a stream of its own and the order between
        # slices is stated by events (below).  NCCL runs a group's collectives one after another
        # in issue order whatever stream they were issued on, so there two streams are enough.
        per_slice = pieces if dv["barriers"] is not None else 2
        streams = self._streams(x.device, per_slice) if pieces > 1 else [torch.cuda.current_stream()]
        main = torch.cuda.current_stream()
        routed = []
        # The slices form a pipeline: slice p's rows cross the links while slice p-1 is
        # multiplied, and slice p-1's results come back while slice p is multiplied.  Two
        # rules keep it one: a slice's dispatch starts when the previous slice's has left
        # (two dispatches at once only halve each other's link rate and finish together,
        # after which nothing is left to hide behind the GEMMs), and a slice's GEMMs start
        # when the previous slice's are done (so its results can start home at once).
        pushed, multiplied = [], []
        # Stage 1, every slice: route, plan, push, barrier.  Issued for all slices before
        # any GEMM so that the collectives (which NCCL runs in issue order) of a later
        # slice are not queued behind an earlier slice's post-GEMM barrier.
        for p, (start, rows) in enumerate(slices):
            sl = slice(start, start + rows)
            st = streams[p % len(streams)]
            if st is not main:
                st.wait_stream(main)
            with torch.cuda.stream(st):
                r = self.ops.route(scores[sl].contiguous(), self.top_k, scores_are_logits)
                bar = dv["barriers"][p] if dv["barriers"] is not None else None
                if bar is not None:
                    allc = bar.all_gather_i32(r.accepted_counts)
                else:
                    allc = torch.empty((self.world, self.experts), dtype=torch.int32, device=x.device)
                    dist.all_gather_into_tensor(allc, r.accepted_counts, group=self.group)
                dst_base, offsets, index = self.ops.ep_plan(allc, self.world, self.rank, self.experts)
                back = (self.ops.ep_return_plan(allc, self.world, self.rank, self.experts)
                        if self.return_path == "push" else ())
                if pushed:
                    st.wait_event(pushed[-1])
                self._size_exchange(alone=(p == 0))
                self.ops.ep_push(x[sl], r, dst_base, dv["ptrs_in"][p], caps[p], self.world, self.experts)
                pushed.append(torch.cuda.Event())
                pushed[-1].record(st)
                self._sync_ranks(dv, p)                               # every rank's rows have landed
                if st is not main:
                    for tns in (dst_base, offsets, index) + tuple(back) + (() if bar is not None else (allc,)):
                        tns.record_stream(st)
            routed.append((sl, r, dst_base, offsets, index, back))
        # Stage 2, every slice: expert GEMMs on what arrived, barrier, pull + combine.
        for p, (sl, r, dst_base, offsets, index, back) in enumerate(routed):
            st = streams[p % len(streams)]
            with torch.cuda.stream(st):
                inbox = dv["inbox"][first[p]:first[p] + caps[p]]
                hidden = dv["hidden"][first[p]:first[p] + caps[p]]
                res = dv["results"][first[p]:first[p] + caps[p]]
                if multiplied:
                    st.wait_event(multiplied[-1])
                self.ops.grouped_indexed_into(inbox, self.w_up, offsets, index, True, hidden)
                res_in = residual[sl] if residual is not None else None
                if self.return_path == "push":
                    # the down projection sends its rows home from its epilogue; after the
                    # barrier this rank's own buffer holds its tokens' results in its own order
                    rows_back = dv["pair_rows"][p]
                    self.ops.grouped_indexed_peer(hidden, self.w_down, offsets, index, dv["ptrs_back"][p], self.world,
                                                  d_out, rows_back, back[0], back[1])
                    multiplied.append(torch.cuda.Event())
                    multiplied[-1].record(st)
                    self._sync_ranks(dv, p)                           # every rank's results have landed
                    mine = dv["returned"][dv["pair_first"][p]:dv["pair_first"][p] + rows_back]
                    self.ops.combine_into(mine, r, res_in, out[sl])
                else:
                    self.ops.grouped_indexed_into(hidden, self.w_down, offsets, index, False, res)
                    multiplied.append(torch.cuda.Event())
                    multiplied[-1].record(st)
                    self._sync_ranks(dv, p)                           # every rank's results are complete
                    self._size_exchange(alone=(p == pieces - 1))
                    self.ops.ep_pull_combine(dv["ptrs_res"][p], r, dst_base, res_in,
                                             caps[p], self.world, self.experts, d_out, out[sl])
                if st is not main:
                    out.record_stream(st)
        self._size_exchange(alone=True)
        for st in streams:
            if st is not main:
                main.wait_stream(st)
        # `rows_received` stays on the device (one int32 per slice: the last group offset);
        # rows_received() reads it when a report wants it.
        self.last = {"routing": routed[0][1], "pieces": pieces, "exchange": "device", "return_path": self.return_path,
                     "rows_received": None, "rows_sent": n * self.top_k,
                     "group_offsets": [t[3] for t in routed], "accepted_counts": [t[1].accepted_counts for t in routed]}
        return out

    def _size_exchange(self, alone: bool):
        """Grid of the next dispatch / combine kernel (read by the library when it is enqueued)."""
        if self.exchange_ctas:
            if alone:
                self.ops.gemm.set_exchange_ctas(0)
            else:
                self.ops.gemm.set_exchange_ctas(self.exchange_ctas, self.exchange_bulk)

    def _sync_ranks(self, dv, p):
        """Stream-ordered barrier of slice ``p``: the barrier kernel, or a one-element all-reduce."""
        if dv["barriers"] is not None:
            dv["barriers"][p].barrier()
        else:
            dist.all_reduce(dv["token"], group=self.group)

    def rows_sent_remote(self) -> int:
        """Routed rows of the last forward whose expert lives on another rank (synchronises)."""
        local = self.experts // self.world
        total = 0
        for counts in self.last.get("accepted_counts", []):
            c = counts.to(torch.int64)
            total += int((c.sum() - c[self.rank * local:(self.rank + 1) * local].sum()).item())
        return total

    def rows_received(self) -> int:
        """Rows this rank's experts multiplied in the last forward (synchronises when the
        device-driven exchange left the count on the device)."""
        if self.last.get("rows_received") is not None:
            return int(self.last["rows_received"])
        return int(sum(int(o[-1].item()) for o in self.last.get("group_offsets", [])))

    def _forward_peer(self, x, scores, scores_are_logits, residual, out_dtype):
        """Several GPUs, copy-engine exchange.  The tokens go through in ``pieces`` slices:
        first every slice is routed and its rows are pushed into the owners' inboxes;
        then, slice by slice on two streams, the expert GEMMs run on what arrived and the
        results are pushed back, so the pushes of one slice ride under the GEMMs of another."""
        n, d = x.shape
        d_out = self.w_down.shape[2]
        count = self.pieces if isinstance(self.pieces, int) else len(self.pieces)   # equal slices on this path
        pieces = count if (n % count == 0 and n // count >= 256) else 1
        step = n // pieces
        pairs = step * self.top_k
        cap = pairs * min(self.world, 3)                      # inbox rows per slice (3x the even share)
        if self._peer is None or self._peer_shape != (pieces, cap, pairs, d, d_out):
            self._peer = PeerExchange(self.group, x.device, pieces * cap, pieces * pairs, d, d_out)
            self._peer_shape = (pieces, cap, pairs, d, d_out)
        px = self._peer
        local = self.experts // self.world
        main = torch.cuda.current_stream()
        plan = []
        gathered = []
        for p in range(pieces):
            sl = slice(p * step, (p + 1) * step)
            r = self.ops.route(scores[sl].contiguous(), self.top_k, scores_are_logits)
            xp = self.ops.scatter(x[sl], r)
            allc = torch.empty((self.world, self.experts), dtype=torch.int32, device=x.device)
            dist.all_gather_into_tensor(allc, r.accepted_counts, group=self.group)
            plan.append((sl, r, xp, allc))
            gathered.append(allc)
        counts_host = torch.stack(gathered).cpu().to(torch.int64)     # the one host sync of the step
        out = torch.empty((n, d_out), dtype=out_dtype, device=x.device)
        streams = self._streams(x.device)
        work = []
        rows_in = rows_out = 0
        # stage 1: push every slice's rows to their owners (copy engines), then a barrier per slice
        for p, (sl, r, xp, allc) in enumerate(plan):
            send_off, send_rows, inbox_off, back_off, per_dest = exchange_plan(counts_host[p], self.rank, self.world)
            got = int(per_dest[:, self.rank].sum())
            if got > cap:
                raise RuntimeError(f"slice {p}: {got} rows routed to rank {self.rank} exceed the inbox capacity {cap}")
            st = streams[p % 2]
            st.wait_stream(main)
            with torch.cuda.stream(st):
                # destinations in ring order starting after this rank, so that at any moment
                # every GPU is receiving from one sender instead of all senders hitting GPU 0
                for hop in range(self.world):
                    j = (self.rank + 1 + hop) % self.world
                    if send_rows[j]:
                        dst = px.peer_inbox[j][p * cap + inbox_off[j]: p * cap + inbox_off[j] + send_rows[j]]
                        dst.copy_(xp[send_off[j]: send_off[j] + send_rows[j]], non_blocking=True)
                px.barrier()
                xp.record_stream(st)
            work.append((send_off, send_rows, back_off, per_dest, got))
            rows_in += got
            rows_out += int(sum(send_rows))
        # stage 2: expert GEMMs on the rows that arrived, results pushed back, combine
        for p, (sl, r, xp, allc) in enumerate(plan):
            send_off, send_rows, back_off, per_dest, got = work[p]
            st = streams[p % 2]
            with torch.cuda.stream(st):
                # group table of what arrived, built on the host from the counts already there
                flat = counts_host[p][:, self.rank * local:(self.rank + 1) * local].reshape(-1)
                off_host = torch.zeros(flat.numel() + 1, dtype=torch.int32).pin_memory()
                off_host[1:] = torch.cumsum(flat, 0).to(torch.int32)
                offsets = off_host.to(x.device, non_blocking=True)
                index = self._group_index(x.device)
                inbox = px.inbox[p * cap: p * cap + max(got, 1)]
                hidden = self.ops.grouped_indexed(inbox[:got], self.w_up, offsets, index, True)
                y = self.ops.grouped_indexed(hidden, self.w_down, offsets, index, False)
                for hop in range(self.world):
                    s_rank = (self.rank + 1 + hop) % self.world
                    rows = int(per_dest[s_rank, self.rank])
                    if rows:
                        # where my block starts in the sender's permuted order = its send offset for me
                        their_off = int(per_dest[s_rank, :self.rank].sum())
                        dst = px.peer_outbox[s_rank][p * pairs + their_off: p * pairs + their_off + rows]
                        dst.copy_(y[back_off[s_rank]: back_off[s_rank] + rows], non_blocking=True)
                px.barrier()
                yp = px.outbox[p * pairs: (p + 1) * pairs]
                res = residual[sl] if residual is not None else None
                out[sl] = self.ops.combine(yp, r, res, out_dtype)
                for tns in (y, out):
                    tns.record_stream(st)
        for st in streams:
            main.wait_stream(st)
        self.last = {"rows_received": rows_in, "rows_sent": rows_out, "routing": plan[0][1], "pieces": pieces,
                     "exchange": "peer copies"}
        return out

    def _forward_pipelined(self, x, scores, scores_are_logits, residual, out_dtype):
        """Several ranks: the tokens go through in ``pieces`` slices.  Routing and the
        counts exchange of every slice come first (one host sync for all the split
        sizes); then slice i's dispatch / expert GEMMs / combine run on one of two
        streams, so that the all-to-alls of a slice overlap the GEMMs of its
        neighbour."""
        n = x.shape[0]
        count = self.pieces if isinstance(self.pieces, int) else len(self.pieces)   # equal slices on this path
        pieces = count if (n % count == 0 and n // count >= 256) else 1
        step = n // pieces
        on_gpu = x.device.type == "cuda"
        plan = []
        for p in range(pieces):
            sl = slice(p * step, (p + 1) * step)
            r = self.ops.route(scores[sl].contiguous(), self.top_k, scores_are_logits)
            xp = self.ops.scatter(x[sl], r)               # rows sorted by (global) expert = by owner rank
            send, recv = exchange_counts(r.accepted_counts, self.world, self.group)
            plan.append((sl, r, xp, send, recv))
        # the one host sync of the step: every slice's split sizes at once
        sizes = torch.stack([torch.stack([s.sum(1), rv.sum(1)]) for _, _, _, s, rv in plan]).cpu().tolist()
        out = torch.empty((n, self.w_down.shape[2]), dtype=out_dtype, device=x.device)
        streams = self._streams(x.device) if on_gpu and pieces > 1 else [None]
        main = torch.cuda.current_stream() if on_gpu else None
        rows_in = rows_out = 0
        for p, (sl, r, xp, send, recv) in enumerate(plan):
            send_splits = [int(v) for v in sizes[p][0]]
            recv_splits = [int(v) for v in sizes[p][1]]
            stream = streams[p % len(streams)]
            ctx = torch.cuda.stream(stream) if stream is not None else _NullCtx()
            if stream is not None:
                stream.wait_stream(main)
            with ctx:
                got = int(sum(recv_splits))
                recv_x = torch.empty((got, x.shape[1]), dtype=xp.dtype, device=xp.device)
                dist.all_to_all_single(recv_x, xp, output_split_sizes=recv_splits,
                                       input_split_sizes=send_splits, group=self.group)
                offsets, index = received_groups(recv)
                hidden = self.ops.grouped_indexed(recv_x, self.w_up, offsets, index, True)
                y = self.ops.grouped_indexed(hidden, self.w_down, offsets, index, False)
                yp = torch.empty((xp.shape[0], y.shape[1]), dtype=y.dtype, device=y.device)
                dist.all_to_all_single(yp, y, output_split_sizes=send_splits, input_split_sizes=recv_splits,
                                       group=self.group)
                res = residual[sl] if residual is not None else None
                out[sl] = self.ops.combine(yp, r, res, out_dtype)
                if stream is not None:
                    for tns in (xp, out):
                        tns.record_stream(stream)
            rows_in += got
            rows_out += int(sum(send_splits))
        if streams[0] is not None:
            for st in streams:
                main.wait_stream(st)
        self.last = {"rows_received": rows_in, "rows_sent": rows_out, "routing": plan[0][1], "pieces": pieces}
        return out

    def _group_index(self, device):
        if self._index is None:
            local = self.experts // self.world
            self._index = torch.arange(local, dtype=torch.int32, device=device).repeat(self.world)
        return self._index

    def _streams(self, device, count: int = 2):
        if self._side is None:
            self._side = []
        while len(self._side) < count:
            self._side.append(torch.cuda.Stream(device=device))
        return self._side[:count]


class _NullCtx:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


class PeerExchange:
    """Row exchange between the GPUs of one box by copy-engine pushes into peer memory.

    Each rank owns two buffers that every peer can write (``torch.distributed``
    symmetric memory: ordinary device memory mapped into the peers' address
    spaces).  A dispatch is a handful of ``cudaMemcpyAsync`` calls per rank: the
    copy engines move the rows over NVLink while the SMs keep multiplying, which
    an all-to-all made of NCCL kernels cannot do next to a persistent GEMM that
    occupies every SM.  Ordering between ranks comes from one-element NCCL
    all-reduces used as stream-ordered barriers; no kernel here spins on a
    peer's flag and no kernel reads peer memory."""

    def __init__(self, group, device, rows_in, rows_back, d_in, d_back, dtype=torch.bfloat16):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.rows_in, self.rows_back = rows_in, rows_back
        self.inbox = symm_mem.empty((rows_in, d_in), dtype=dtype, device=device)        # rows dispatched to me
        self.outbox = symm_mem.empty((rows_back, d_back), dtype=dtype, device=device)   # results returned to me
        name = self.group.group_name
        self._in = symm_mem.rendezvous(self.inbox, name)
        self._back = symm_mem.rendezvous(self.outbox, name)
        self.peer_inbox = [self._in.get_buffer(r, (rows_in, d_in), dtype) for r in range(self.world)]
        self.peer_outbox = [self._back.get_buffer(r, (rows_back, d_back), dtype) for r in range(self.world)]
        self._token = torch.zeros(1, device=device)

    def barrier(self):
        """Stream-ordered: later work on this stream starts after every rank got here."""
        dist.all_reduce(self._token, group=self.group)


class PeerBarrier:
    """Stream-ordered barrier between the GPUs of one box, made of one tiny kernel per rank.

    Each rank owns ``world`` arrival words in symmetric memory.  ``barrier()`` launches a
    one-block kernel on the current stream that writes this rank's epoch into its word on
    every peer and waits (bounded) until all of its own words reached the epoch.  The kernel
    uses no shared memory and fits on an SM beside a persistent GEMM CTA, so it neither waits
    for the GEMM to finish nor needs SMs kept free, which a one-element NCCL all-reduce does;
    it costs a launch and one NVLink round trip.  ``all_gather_i32`` gathers a few integers
    per rank on the way (the expert-parallel exchange's per-expert counts).

    Every rank must call the same sequence on ONE stream per object (epochs count up); a
    wait that runs out leaves device status 108 on the handle and the object unusable."""

    def __init__(self, ops, group, device, payload_count: int = 0, limit_ms: int = 2000):
        import ctypes as C
        import torch.distributed._symmetric_memory as symm_mem
        self.ops = ops
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.limit_ms, self.count, self.epoch = limit_ms, payload_count, 0
        name = self.group.group_name
        self._words = symm_mem.empty((self.world,), dtype=torch.int64, device=device)
        self._words.zero_()
        self._h_words = symm_mem.rendezvous(self._words, name)
        self._ptr_words = (C.c_void_p * self.world)()
        for r in range(self.world):
            self._ptr_words[r] = self._h_words.get_buffer(r, (self.world,), torch.int64).data_ptr()
        self._ptr_tables = None
        if payload_count:
            shape = (2, self.world, payload_count)
            self._table = symm_mem.empty(shape, dtype=torch.int32, device=device)
            self._h_table = symm_mem.rendezvous(self._table, name)
            self._ptr_tables = (C.c_void_p * self.world)()
            for r in range(self.world):
                self._ptr_tables[r] = self._h_table.get_buffer(r, shape, torch.int32).data_ptr()
        # no peer may write an arrival word before every rank has zeroed its own
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)

    def barrier(self):
        self.epoch += 1
        self.ops.peer_barrier(self._ptr_words, self.world, self.rank, self.epoch, self.limit_ms)

    def all_gather_i32(self, mine):
        """Every rank's ``mine`` (int32, ``payload_count`` long) as ``[world, payload_count]``: a
        view of this rank's table, valid until the second next call."""
        if mine.numel() != self.count or mine.dtype != torch.int32:
            raise ValueError("payload must be payload_count int32")
        self.epoch += 1
        self.ops.peer_barrier(self._ptr_words, self.world, self.rank, self.epoch, self.limit_ms, mine,
                              self._ptr_tables)
        return self._table[self.epoch & 1]


def exchange_plan(counts_all, rank, world):
    """Offsets of a dispatch from the full counts matrix ``counts_all[src, expert]`` (host ints).

    Returns ``(send_off, send_rows, inbox_off, back_off)``: my rows for rank j start at
    ``send_off[j]`` of my permuted buffer and land at ``inbox_off[j]`` of j's inbox (after
    the rows of lower-ranked sources); rank s's rows sit at ``back_off[s]`` of my inbox."""
    experts = counts_all.shape[1]
    local = experts // world
    per_dest = counts_all.reshape(world, world, local).sum(2)          # [src, dest]
    send_rows = per_dest[rank].tolist()
    send_off = [int(v) for v in (per_dest[rank].cumsum(0) - per_dest[rank]).tolist()]
    before = per_dest.cumsum(0) - per_dest                              # rows of lower-ranked sources, per dest
    inbox_off = [int(before[rank, j]) for j in range(world)]
    back_off = [int(before[s, rank]) for s in range(world)]
    return send_off, [int(v) for v in send_rows], inbox_off, back_off, per_dest


class PeerRowExchange:
    """Reduce-scatter and all-gather of row blocks by copy-engine pushes into peer memory.

    A reduce-scatter made of NCCL kernels needs SMs, and next to a persistent GEMM that holds
    every SM it gets few of them, late (measured at 8 GPUs: 0.45 ms per 134 MB piece, a third of
    the link rate, while the GEMMs it ran beside slowed down too).  Here every rank instead
    *copies* the row block each peer owns straight into that peer's inbox (``cudaMemcpyAsync``
    between peer-mapped buffers: the copy engines move the bytes over NVLink, no SM is
    involved), a barrier orders the ranks, and a small kernel of this library
    adds the ``world`` parts that arrived (fp32 adds, rank order).  The all-gather is the same
    without the sum.  Buffers are ``torch.distributed`` symmetric memory; the row data moves by
    copy engine only, and the ranks wait for one another in a one-block barrier kernel
    (``PeerBarrier``, bounded wait) or, on request, a one-element all-reduce."""

    def __init__(self, ops, group, device, shares, width, dtype=torch.bfloat16, barrier="kernel"):
        """``shares[s]`` = rows every rank owns in slot ``s`` (slots may differ in size).
        ``barrier``: "kernel" = this library's barrier kernel (``PeerBarrier``), "nccl" = a
        one-element all-reduce."""
        import torch.distributed._symmetric_memory as symm_mem
        self.ops = ops
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.shares, self.width = list(shares), width
        sizes = [self.world * sh * width for sh in self.shares]
        self._off = [sum(sizes[:i]) for i in range(len(sizes))]
        total = sum(sizes)
        self._inbox = symm_mem.empty((total,), dtype=dtype, device=device)       # parts of the rows I own
        self._gathered = symm_mem.empty((total,), dtype=dtype, device=device)    # every rank's rows, in rank order
        name = self.group.group_name
        self._h_in = symm_mem.rendezvous(self._inbox, name)
        self._h_all = symm_mem.rendezvous(self._gathered, name)
        self._peer_inbox = [self._h_in.get_buffer(r, (total,), dtype) for r in range(self.world)]
        self._peer_gathered = [self._h_all.get_buffer(r, (total,), dtype) for r in range(self.world)]
        self._token = torch.zeros(1, device=device)
        self._barrier = PeerBarrier(ops, self.group, device) if barrier == "kernel" else None

    def _slot(self, flat, slot):
        """``[world, share, width]`` view of slot ``slot`` of a flat buffer."""
        sh = self.shares[slot]
        n = self.world * sh * self.width
        return flat[self._off[slot]:self._off[slot] + n].view(self.world, sh, self.width)

    def barrier(self):
        """Stream-ordered: what follows on this stream starts after every rank got here."""
        if self._barrier is not None:
            self._barrier.barrier()
        else:
            dist.all_reduce(self._token, group=self.group)

    def reduce_scatter(self, slot, partial, out):
        """``out [share, width] = sum over ranks of their partial[rank_rows]``; ``partial`` is
        ``[world * share, width]``.  Runs on the current stream."""
        sh = self.shares[slot]
        # ring order starting after this rank: at any moment every GPU receives from one sender
        for hop in range(self.world):
            j = (self.rank + 1 + hop) % self.world
            self._slot(self._peer_inbox[j], slot)[self.rank].copy_(partial[j * sh:(j + 1) * sh], non_blocking=True)
        self.barrier()
        self.ops.sum_parts(self._slot(self._inbox, slot), out)
        return out

    def all_gather(self, slot, mine):
        """Every rank's ``mine [share, width]`` in rank order: returns a ``[world * share, width]``
        view of this rank's buffer, valid until ``slot`` is used again."""
        for hop in range(self.world):
            j = (self.rank + 1 + hop) % self.world
            self._slot(self._peer_gathered[j], slot)[self.rank].copy_(mine, non_blocking=True)
        self.barrier()
        return self._slot(self._gathered, slot).view(self.world * self.shares[slot], self.width)


# --------------------------------------------------------------------------- tensor-parallel MLP

class TensorParallelMlp:
    """Column-parallel ``up`` ([d, ff / world]) and row-parallel ``down`` ([ff / world, d]).

    ``forward`` takes the replicated ``x [m, d]`` and returns this rank's rows of
    ``y = (x . W_up) . W_down`` after a reduce-scatter.  Rows are processed in pieces; the
    reduce-scatter of a piece runs on a side stream while the next piece's GEMMs run, and of
    every piece ``[start, start + rows)`` rank ``r`` ends up owning rows
    ``[start + r * rows / world, start + (r + 1) * rows / world)``.

    ``chunks`` is the number of equal pieces, or a list of row fractions (e.g.
    ``[1, 3, 4, 4, 3, 1]``): what no GEMM can cover is the exchange of the LAST piece of the
    forward and of the backward and the gather of the backward's FIRST piece, so short pieces
    at both ends shorten exactly that, while the long ones in the middle keep the GEMMs large."""

    def __init__(self, ops, w_up_shard, w_down_shard, group=None, chunks=4,
                 partial_dtype=torch.bfloat16, reserve_sms: int = 0, exchange: str = "nccl",
                 barrier: str = "kernel"):
        self.ops, self.group, self.chunks = ops, group, chunks
        self.barrier = barrier              # how the copy exchange orders the ranks (PeerRowExchange)
        self.reserve_sms = reserve_sms      # SMs every GEMM leaves to the collectives on the side stream
        self.world, self.rank = _world(group)
        self.w_up, self.w_down = w_up_shard, w_down_shard
        self.partial_dtype = partial_dtype
        self._comm_stream = None
        # "nccl": reduce_scatter_tensor / all_gather_into_tensor; "copy": copy-engine pushes into
        # peer memory + a local sum (PeerRowExchange), CUDA tensors and more than one rank only
        self.exchange, self._px, self._px_key = exchange, None, None
        self._bufs = {}

    def pieces(self, m: int):
        """``[(first row, rows), ...]`` of the pieces ``m`` rows are processed in."""
        if isinstance(self.chunks, int):
            if m % (self.chunks * self.world):
                raise ValueError("rows must divide by chunks * world")
            return [(c * (m // self.chunks), m // self.chunks) for c in range(self.chunks)]
        total = sum(self.chunks)
        rows = [m * f // total for f in self.chunks]
        if sum(rows) != m or any(r <= 0 or r % self.world for r in rows):
            raise ValueError("every piece must be a positive multiple of the world size and the pieces must add up")
        starts = [sum(rows[:i]) for i in range(len(rows))]
        return list(zip(starts, rows))

    def _peer(self, x, plan):
        """The copy-engine exchange for this problem size, or None (NCCL / gloo path)."""
        if self.exchange != "copy" or x.device.type != "cuda" or self.world == 1:
            return None
        key = (tuple(plan), x.shape[1], self.partial_dtype)
        if self._px is None or self._px_key != key:
            if self.w_down.shape[1] != x.shape[1]:
                raise ValueError("the copy exchange needs the MLP's input and output widths to match")
            self._px = PeerRowExchange(self.ops, self.group, x.device, [rows // self.world for _, rows in plan],
                                       x.shape[1], self.partial_dtype, barrier=self.barrier)
            self._px_key = key
        return self._px

    def _buf(self, name, shape, dtype, device):
        """A buffer this object keeps between steps (CUDA): a step in steady state allocates
        nothing, so the caching allocator never has to grow -- or call cudaMalloc -- while the
        host runs several steps ahead of the GPU.  What ``forward`` / ``backward`` return lives
        in such buffers and is valid until the next call of the same method."""
        if device.type != "cuda":
            return torch.empty(shape, dtype=dtype, device=device)
        key = (name, tuple(shape), dtype)
        t = self._bufs.get(key)
        if t is None:
            t = self._bufs[key] = torch.empty(shape, dtype=dtype, device=device)
        return t

    def _side_stream(self, device):
        if device.type != "cuda":
            return None
        if self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=device)
        return self._comm_stream

    def owned_rows(self, m: int):
        """Global row indices this rank holds after ``forward`` (in output order)."""
        idx = []
        for start, rows in self.pieces(m):
            share = rows // self.world
            idx.append(torch.arange(start + self.rank * share, start + (self.rank + 1) * share))
        return torch.cat(idx)

    def forward(self, x):
        with _ReservedSms(self.ops, self.reserve_sms if self.world > 1 else 0):
            return self._forward(x)

    def backward(self, x, dy_local, dw_up, dw_down):
        """``dy_local`` is this rank's rows of dL/dy (layout of ``forward``'s output).

        Accumulates the weight-gradient shards (fp32) and returns this rank's rows
        of ``dx`` (same row ownership as ``forward``'s output) after a
        reduce-scatter -- the mirror image of the all-gather that hands the MLP its
        replicated ``x``.  Piece by piece: the all-gather of the next piece's ``dy``
        and the reduce-scatter of the previous piece's ``dx`` run on a side stream
        underneath the current piece's four GEMMs."""
        with _ReservedSms(self.ops, self.reserve_sms if self.world > 1 else 0):
            return self._backward(x, dy_local, dw_up, dw_down)

    def _forward(self, x):
        m, d = x.shape[0], self.w_down.shape[1]
        plan = self.pieces(m)
        out = self._buf("y", (m // self.world, d), self.partial_dtype, x.device)
        side = self._side_stream(x.device)
        px = self._peer(x, plan)
        self._hidden = []
        done = 0
        ff_local = self.w_up.shape[1]
        fused = hasattr(self.ops, "gemm")                    # the device ops take output buffers
        for c, (start, rows) in enumerate(plan):
            share = rows // self.world
            xs = x[start:start + rows]
            if fused:
                h = self.ops.linear(xs, self.w_up, torch.bfloat16,
                                    out=self._buf(("h", c), (rows, ff_local), torch.bfloat16, x.device))
                y = self.ops.linear(h, self.w_down, self.partial_dtype,
                                    out=self._buf(("partial", c), (rows, d), self.partial_dtype, x.device))
            else:
                h = self.ops.linear(xs, self.w_up, torch.bfloat16)
                y = self.ops.linear(h, self.w_down, self.partial_dtype)
            self._hidden.append(h)
            dst = out[done:done + share]
            done += share
            if side is None:
                dist.reduce_scatter_tensor(dst, y, op=dist.ReduceOp.SUM, group=self.group)
            else:
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    if px is not None:
                        px.reduce_scatter(c, y, dst)
                    else:
                        dist.reduce_scatter_tensor(dst, y, op=dist.ReduceOp.SUM, group=self.group)
                if not fused:
                    y.record_stream(side)
        if side is not None:
            torch.cuda.current_stream().wait_stream(side)
        return out

    def _backward(self, x, dy_local, dw_up, dw_down):
        m = x.shape[0]
        plan = self.pieces(m)
        first = [sum(rows // self.world for _, rows in plan[:c]) for c in range(len(plan))]   # of my rows, per piece
        dx = self._buf("dx_partial", (m, x.shape[1]), self.partial_dtype, x.device)
        dx_local = self._buf("dx", (m // self.world, x.shape[1]), self.partial_dtype, x.device)
        side = self._side_stream(x.device)
        main = torch.cuda.current_stream() if side is not None else None
        fused = hasattr(self.ops, "gemm")
        px = self._peer(x, plan) if dy_local.dtype == self.partial_dtype else None

        def gather(c):
            rows = plan[c][1]
            share = rows // self.world
            src = dy_local[first[c]:first[c] + share].contiguous()
            if px is not None:
                with torch.cuda.stream(side):
                    dy = px.all_gather(c, src)
                    done = torch.cuda.Event()
                    done.record(side)
                return dy, done
            dy = self._buf(("dy", c), (rows, dy_local.shape[1]), dy_local.dtype, x.device)
            if side is None:
                dist.all_gather_into_tensor(dy, src, group=self.group)
                return dy, None
            with torch.cuda.stream(side):
                dist.all_gather_into_tensor(dy, src, group=self.group)
                done = torch.cuda.Event()
                done.record(side)
            return dy, done

        if side is not None:
            side.wait_stream(main)
        nxt = gather(0)
        for c, (start, rows) in enumerate(plan):
            share = rows // self.world
            dy, ready = nxt
            if c + 1 < len(plan):
                nxt = gather(c + 1)                                       # prefetch under this piece's GEMMs
            if ready is not None:
                main.wait_event(ready)
            h = self._hidden[c]
            self.ops.linear_weight_grad(h, dy, dw_down)                   # dW_down += h^T dy
            if fused:                                                     # dh = dy W_down^T
                dh = self.ops.linear_input_grad(dy, self.w_down, torch.bfloat16,
                                                out=self._buf("dh", (rows, self.w_down.shape[0]), torch.bfloat16,
                                                              x.device))
            else:
                dh = self.ops.linear_input_grad(dy, self.w_down, torch.bfloat16)
            xs = x[start:start + rows]
            self.ops.linear_weight_grad(xs, dh, dw_up)                    # dW_up += x^T dh
            dxs = dx[start:start + rows]
            self.ops.linear_input_grad_into(dh, self.w_up, dxs)           # dx piece (partial sum)
            mine = dx_local[first[c]:first[c] + share]
            if side is None:
                dist.reduce_scatter_tensor(mine, dxs, op=dist.ReduceOp.SUM, group=self.group)
            else:
                produced = torch.cuda.Event()
                produced.record(main)
                with torch.cuda.stream(side):
                    side.wait_event(produced)
                    if px is not None:
                        px.reduce_scatter(c, dxs, mine)
                    else:
                        dist.reduce_scatter_tensor(mine, dxs, op=dist.ReduceOp.SUM, group=self.group)
        if side is not None:
            main.wait_stream(side)
        return dx_local
