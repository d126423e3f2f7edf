"""Expert-parallel MoE-block forward over the ranks of one node.

The reference is single-GPU (its design notes name expert parallelism with an
NCCL all-to-all as future work); this module adds it around the same CUDA
stages.  Rank ``r`` of ``G`` owns experts ``[r*E/G, (r+1)*E/G)`` and brings its
own tokens.  One step:

1. route the local tokens, plan the local permutation (rows sorted by global
   expert id, hence by destination rank);
2. exchange per-expert row counts and activation maxima (one small all-gather)
   so that every rank derives the same per-expert FP8 scale a single GPU
   would;
3. quantise the local rows with those scales and send them to the owners of
   their experts (dispatch all-to-all, FP8 payload);
4. regroup the received rows into per-expert segments ordered by (source rank,
   source row) - the order a single GPU would have - and run gate/up + SwiGLU,
   requant and the down projection on the local experts;
5. send the bf16 result rows back (combine all-to-all) and do the weighted
   top-k combine at home.

The result is bit-identical to the single-GPU forward over the concatenated
tokens.  The index arithmetic (:class:`ExchangePlan`, :func:`dispatch`,
:func:`combine_back`) is device-agnostic torch code and is tested on CPU with
``gloo``; the compute stages exist on CUDA only.
"""

from __future__ import annotations

import ctypes as C
import os
import warnings

import torch
import torch.distributed as dist

from . import _lib

_FP8 = torch.float8_e4m3fn


class ExchangePlan:
    """Split sizes and row maps of one dispatch/combine pair, derived from the
    ``[G, E]`` matrix of per-rank, per-expert row counts."""

    def __init__(self, counts: torch.Tensor, rank: int, counts_host: torch.Tensor = None):
        G, E = counts.shape
        assert E % G == 0, (E, G)
        self.rank, self.world, self.experts_local = rank, G, E // G
        el = self.experts_local
        # the only host copy: split sizes must be ints (callers planning several exchanges pass one copy)
        cpu = (counts.cpu() if counts_host is None else counts_host).to(torch.int64)
        self.send_splits = cpu[rank].view(G, el).sum(1).tolist()  # rows I send to each rank
        mine = cpu[:, rank * el:(rank + 1) * el]                 # [G, el] rows each rank sends me, per local expert
        self.recv_splits = mine.sum(1).tolist()
        self.rows_local = int(mine.sum())
        dev = counts.device
        mine = mine.to(dev)
        # received order is (source, expert); wanted order is (expert, source)
        start_src = (torch.cumsum(mine.reshape(-1), 0) - mine.reshape(-1)).view(G, el)
        sizes_dst = mine.t().reshape(-1)                         # blocks in (expert, source) order
        start_dst = torch.cumsum(sizes_dst, 0) - sizes_dst
        block_src = start_src.t().reshape(-1)
        n = self.rows_local
        rows = torch.arange(n, device=dev)
        self.src_of_dst = (torch.repeat_interleave(block_src - start_dst, sizes_dst, output_size=n) + rows)
        self.dst_of_src = torch.empty_like(self.src_of_dst)      # inverse map: the way back is a gather too
        self.dst_of_src[self.src_of_dst] = rows
        seg = mine.sum(0)
        self.offsets = torch.zeros(el + 1, dtype=torch.int32, device=dev)
        self.offsets[1:] = torch.cumsum(seg, 0).to(torch.int32)
        self.row_expert = torch.repeat_interleave(torch.arange(el, device=dev, dtype=torch.int32), seg, output_size=n)


def dispatch(rows: torch.Tensor, plan: ExchangePlan, group=None) -> torch.Tensor:
    """Send rows (sorted by global expert id) to the expert owners; returns the
    received rows regrouped into per-local-expert segments."""
    recv = rows.new_empty((plan.rows_local,) + tuple(rows.shape[1:]))
    dist.all_to_all_single(recv, rows, plan.recv_splits, plan.send_splits, group=group)
    if plan.experts_local == 1:           # one expert per rank: (source, expert) order is already (expert, source)
        return recv
    return recv.index_select(0, plan.src_of_dst)


def dispatch_start(rows: torch.Tensor, plan: ExchangePlan, group=None):
    """Asynchronous half of :func:`dispatch`: returns ``(recv, work)``; after ``work.wait()`` pass
    ``recv`` to :func:`dispatch_finish`."""
    recv = rows.new_empty((plan.rows_local,) + tuple(rows.shape[1:]))
    work = dist.all_to_all_single(recv, rows, plan.recv_splits, plan.send_splits, group=group, async_op=True)
    return recv, work


def dispatch_finish(recv: torch.Tensor, plan: ExchangePlan) -> torch.Tensor:
    return recv if plan.experts_local == 1 else recv.index_select(0, plan.src_of_dst)


def combine_back_start(rows_local: torch.Tensor, plan: ExchangePlan, n_home: int, group=None):
    """Asynchronous :func:`combine_back`: returns ``(home, work)``."""
    send = rows_local if plan.experts_local == 1 else rows_local.index_select(0, plan.dst_of_src)
    home = rows_local.new_empty((n_home,) + tuple(rows_local.shape[1:]))
    work = dist.all_to_all_single(home, send, plan.send_splits, plan.recv_splits, group=group, async_op=True)
    return home, work


def combine_back(rows_local: torch.Tensor, plan: ExchangePlan, n_home: int, group=None) -> torch.Tensor:
    """Inverse of :func:`dispatch`: per-expert rows go back to the ranks (and row
    positions) they came from."""
    send = rows_local if plan.experts_local == 1 else rows_local.index_select(0, plan.dst_of_src)
    home = rows_local.new_empty((n_home,) + tuple(rows_local.shape[1:]))
    dist.all_to_all_single(home, send, plan.send_splits, plan.recv_splits, group=group)
    return home


class ExpertParallelMoE:
    """Holds this rank's expert shard and runs the expert-parallel forward."""

    def __init__(self, w_gate, experts_w_gate, experts_w_up, experts_w_down, scales_gate, scales_up, scales_down,
                 num_experts: int, top_k: int, group=None, max_tokens_per_rank: int = None):
        """``max_tokens_per_rank``: the largest batch any rank will ever bring (the same value on every rank).
        The peer-memory transport sizes its receive buffers from it, for the worst case of every row of every
        rank landing on one rank.  Without it the ranks agree on the largest batch of their FIRST forward;
        ranks may bring different numbers of tokens, but none may later exceed the agreed figure."""
        self.group = group
        self.max_tokens_per_rank = max_tokens_per_rank
        self._agreed_tokens = None
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.E, self.K = num_experts, top_k
        assert num_experts % self.world == 0
        self.el = num_experts // self.world
        assert experts_w_gate.shape[0] == self.el, "pass this rank's expert shard"
        self.w_gate = w_gate.contiguous()
        self.wg, self.wu, self.wd = (t.contiguous() for t in (experts_w_gate, experts_w_up, experts_w_down))
        self.sg, self.su, self.sd = (t.to(torch.float32).contiguous() for t in (scales_gate, scales_up, scales_down))
        self.block = self.sg.dim() == 3          # [E_local, in/128, out/128] inverse scales: block recipe
        self.D, self.H = self.wg.shape[1], self.wg.shape[2]
        self.dev = self.wg.device
        assert self.w_gate.shape == (self.D, num_experts)

    #: token micro-batches per forward: the dispatch of batch i+1 overlaps the gate/up GEMM of batch i and
    #: the way back of batch i overlaps the down GEMM of batch i+1.  Results do not depend on it.
    micro_batches = 1
    micro_batch_min_tokens = 2048      # smaller batches per rank are not split
    #: SMs the persistent GEMMs leave to NCCL while micro-batches overlap (they otherwise hold every SM
    #: until they finish, and the collective queued beside them cannot start)
    sm_reserve = 0
    #: "nccl": all-to-all over NCCL plus a row regroup on either side.  "peer": the quantisation kernel stores
    #: each row straight into its owner's memory and the combine kernel loads result rows from their owners'
    #: memory (symmetric memory over NVLink, three stream-ordered barriers per step, no collective on the
    #: data path).  "auto": "peer" where symmetric memory can be set up (per-tensor recipe, CUDA, <= 8 ranks).
    transport = "auto"
    #: way back of the peer transport.  "push": the down projection's epilogue stores each finished row
    #: into its home rank's buffer (the transfer overlaps the GEMM) and the combine is local.  "pull": the
    #: down projection writes locally and the combine kernel loads the rows from their owners.
    #: The epilogue transposes its stores so that each one writes 128 contiguous bytes of a row (with one
    #: 16-byte store per lane the rows crossed NVLink at ~140 GB/s and the GEMM waited for them).
    way_back = "push"

    def _push(self) -> bool:
        return self.way_back != "pull"

    _peer = None
    #: [ranks, experts] row counts of the last peer-memory step (device tensor; None before the first step)
    last_counts = None
    #: when True, the peer-memory forward records a CUDA event at every phase boundary;
    #: :meth:`phase_times` turns the last step's events into milliseconds
    profile = False
    _marks = ()

    def _mark(self, name: str):
        if self.profile:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(torch.cuda.current_stream(self.dev))
            self._marks.append((name, ev))

    def phase_times(self) -> dict:
        """Milliseconds between the phase marks of the last profiled step (synchronises)."""
        torch.cuda.synchronize(self.dev)
        m = self._marks
        return {m[i + 1][0]: m[i][1].elapsed_time(m[i + 1][1]) for i in range(len(m) - 1)}

    def _peer_setup(self, rows_cap: int):
        """Symmetric receive (FP8 rows) and result (bf16 rows) buffers of ``rows_cap`` rows, mapped on every rank.
        Collective.  Returns False (on every rank alike) when symmetric memory is not available."""
        if self._peer is not None and self._peer["cap"] >= rows_cap:
            return True
        if self._peer is False:
            return False
        ok = 1
        try:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")     # plain peer loads/stores only
            import torch.distributed._symmetric_memory as symm
            group = self.group if self.group is not None else dist.group.WORLD
            xq = symm.empty(rows_cap * self.D, dtype=torch.uint8, device=self.dev)
            y = symm.empty(rows_cap * self.D, dtype=torch.bfloat16, device=self.dev)
            hx, hy = symm.rendezvous(xq, group), symm.rendezvous(y, group)
            G = self.world
            peer = dict(cap=rows_cap, xq=xq, y=y, hx=hx, hy=hy,
                        xq_ptrs=(C.c_void_p * G)(*[int(p) for p in hx.buffer_ptrs]),
                        y_ptrs=(C.c_void_p * G)(*[int(p) for p in hy.buffer_ptrs]))
            if self.block:               # per-row group scales travel with the codes
                xinv = symm.empty(rows_cap * ((self.D + 127) // 128), dtype=torch.float32, device=self.dev)
                hi = symm.rendezvous(xinv, group)
                peer.update(xinv=xinv, hi=hi, xinv_ptrs=(C.c_void_p * G)(*[int(p) for p in hi.buffer_ptrs]))
        except Exception as ex:      # noqa: BLE001 - any failure means "use NCCL", agreed on below
            ok, peer = 0, repr(ex)
        flag = torch.tensor([ok], dtype=torch.int32, device=self.dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 0:
            if self.rank == 0:
                warnings.warn(f"expert parallelism: symmetric memory unavailable ({peer if not ok else 'on a peer'}); "
                              "using the NCCL all-to-all transport")
            self._peer = False
            return False
        self._peer = peer
        return True

    def _agree_on_capacity(self, T: int) -> int:
        """Row capacity of every rank's receive buffer, decided once by all ranks together: the largest batch
        any rank declared (or brought to this first forward), times ranks, times top_k.  A rank never decides
        alone to enter the collective set-up, and a later batch above the agreed size is refused before any
        collective of that step is issued."""
        if self._agreed_tokens is None:
            t = torch.tensor([max(T, self.max_tokens_per_rank or 0)], dtype=torch.int64, device=self.dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
            self._agreed_tokens = int(t.item())
        if T > self._agreed_tokens:
            raise ValueError(f"this rank brings {T} tokens but the ranks agreed on at most {self._agreed_tokens} per rank; "
                             "construct ExpertParallelMoE with max_tokens_per_rank (the same value on every rank)")
        return self.world * self._agreed_tokens * self.K

    def _use_peers(self, T: int) -> bool:
        if self.transport == "nccl" or self.dev.type != "cuda" or self.world > 8:
            return False
        ok = self._peer_setup(self._agree_on_capacity(T))    # worst case: every row of every rank lands here
        if not ok and self.transport == "peer":
            raise RuntimeError("transport='peer' requested but symmetric memory could not be set up")
        return ok

    def _peer_maps(self, counts, offsets):
        """From the [G, E] row counts: where my rows of expert e land on e's owner relative to my own
        permuted order (delta[E]), my local segments, and the way home of the rows I will hold."""
        G, rank, el, E, dev, i32 = self.world, self.rank, self.el, self.E, self.dev, torch.int32
        if dev.type != "cuda":           # the same arithmetic in torch (CPU tests of the protocol)
            total = counts.sum(0, dtype=i32).view(G, el)
            seg_start = (torch.cumsum(total, 1, dtype=i32) - total).view(E)
            below = counts[:rank].sum(0, dtype=i32) if rank > 0 else torch.zeros(E, dtype=i32, device=dev)
            delta = (seg_start + below - offsets[:E]).contiguous()
            offsets_l = torch.zeros(el + 1, dtype=i32, device=dev)
            offsets_l[1:] = torch.cumsum(total[rank], 0, dtype=i32)
            home_counts = counts[:, rank * el:(rank + 1) * el].contiguous()
            home_first = (torch.cumsum(counts, 1, dtype=i32) - counts)[:, rank * el:(rank + 1) * el].contiguous()
            return delta, offsets_l, home_counts, home_first
        buf = torch.empty(E + el + 1 + 2 * G * el, dtype=i32, device=dev)
        delta, offsets_l = buf[:E], buf[E:E + el + 1]
        home_counts, home_first = buf[E + el + 1:E + el + 1 + G * el], buf[E + el + 1 + G * el:]
        _lib.check(_lib.lib().bwmoe_ep_maps(counts.data_ptr(), offsets.data_ptr(), G, E, rank, delta.data_ptr(),
                                            offsets_l.data_ptr(), home_counts.data_ptr(), home_first.data_ptr(),
                                            torch.cuda.current_stream(dev).cuda_stream))
        return delta, offsets_l, home_counts, home_first

    def _forward_block_peers(self, x, weights, indices, host_in):
        """Block-scale recipe over peer memory: tokens are quantised once in token order, their codes and
        group scales stored to the owners; the block GEMMs run locally and the down epilogue stores the
        result rows at home."""
        lib, dev, E, K, D, H, el = _lib.lib(), self.dev, self.E, self.K, self.D, self.H, self.el
        G, rank, T = self.world, self.rank, x.shape[0]
        M = T * K
        st = torch.cuda.current_stream(dev).cuda_stream
        i32, f32, u8 = torch.int32, torch.float32, torch.uint8
        new = lambda *shape, dtype: torch.empty(shape, dtype=dtype, device=dev)      # noqa: E731
        peer = self._peer
        if self.profile:
            self._marks = []
        self._mark("start")
        status = torch.zeros(4, dtype=i32, device=dev)
        offsets, pos, row_slot, row_expert = new(E + 1, dtype=i32), new(M, dtype=i32), new(M, dtype=i32), new(M, dtype=i32)
        scratch = new(lib.bwmoe_plan_scratch_bytes(T, E, K), dtype=u8)
        _lib.check(lib.bwmoe_permute_plan(indices.data_ptr(), None, T, E, K, offsets.data_ptr(), pos.data_ptr(),
                                          row_slot.data_ptr(), row_expert.data_ptr(), None, status.data_ptr(),
                                          scratch.data_ptr(), st))
        nd, nh = (D + 127) // 128, (H + 127) // 128
        xq_tok, inv_tok = new(T, D, dtype=u8), new(T, nd, dtype=f32)
        _lib.check(lib.bwmoe_gather_quant_group(x.data_ptr(), None, T, D, 1, xq_tok.data_ptr(), inv_tok.data_ptr(), st))
        self._mark("plan+quantise")
        counts = new(G * E, dtype=i32)
        dist.all_gather_into_tensor(counts, (offsets[1:] - offsets[:-1]).contiguous(), group=self.group)
        counts = counts.view(G, E)
        self.last_counts = counts                    # [G, E] rows rank s sent to expert e (device tensor)
        delta, offsets_l, home_counts, home_first = self._peer_maps(counts, offsets)
        # No host synchronisation: the number of rows this rank receives stays on the device.  The GEMMs take
        # their tiles from the device-side segment offsets, the buffers are sized for the agreed worst case,
        # and a row beyond it is dropped by the store kernel (status bit), never written past the buffer.
        cap = peer["cap"]
        self._mark("counts+maps")
        peer["hx"].barrier()
        self._mark("barrier A")
        _lib.check(lib.bwmoe_scatter_rows_group_peers(xq_tok.data_ptr(), inv_tok.data_ptr(), pos.data_ptr(),
                                                      indices.data_ptr(), delta.data_ptr(), T, D, K, el,
                                                      peer["xq_ptrs"], peer["xinv_ptrs"], G, cap, status.data_ptr(), st))
        self._mark("store rows")
        peer["hx"].barrier()
        self._mark("barrier B")
        if "hq" not in peer:
            peer["hq"], peer["h_inv"] = new(cap, H, dtype=u8), new(cap, nh, dtype=f32)
        hq, h_inv = peer["hq"], peer["h_inv"]
        xinv_l = peer["xinv"]
        if not 3 <= nd <= 16:
            # The GEMM stages a tile's scales in shared memory (read once per tile) only for 3..16 K blocks;
            # otherwise its fold warps re-read them per K block and rely on L1, which loads from peer-mapped
            # memory were measured not to get: copy them into ordinary device memory first.
            xinv_l = peer["xinv"].clone()
            self._mark("copy scales")
        _lib.check(lib.bwmoe_gateup_swiglu_block(peer["xq"].data_ptr(), xinv_l.data_ptr(), offsets_l.data_ptr(),
                                                 self.wg.data_ptr(), self.wu.data_ptr(), self.sg.data_ptr(),
                                                 self.su.data_ptr(), cap, D, H, el, hq.data_ptr(), h_inv.data_ptr(),
                                                 status.data_ptr(), st))
        self._mark("gate/up")
        if self._push():
            _lib.check(lib.bwmoe_down_block_peers(hq.data_ptr(), h_inv.data_ptr(), offsets_l.data_ptr(),
                                                  self.wd.data_ptr(), self.sd.data_ptr(), cap, D, H, el,
                                                  home_counts.data_ptr(), home_first.data_ptr(), peer["y_ptrs"],
                                                  G, status.data_ptr(), st))
        else:
            _lib.check(lib.bwmoe_down_block(hq.data_ptr(), h_inv.data_ptr(), offsets_l.data_ptr(),
                                            self.wd.data_ptr(), self.sd.data_ptr(), cap, D, H, el,
                                            peer["y"].data_ptr(), status.data_ptr(), st))
        self._mark("down")
        peer["hy"].barrier()
        self._mark("barrier C")
        out = new(T, D, dtype=torch.bfloat16)
        if self._push():
            _lib.check(lib.bwmoe_combine(peer["y"].data_ptr(), pos.data_ptr(), weights.data_ptr(), T, D, K,
                                         out.data_ptr(), st))
        else:
            _lib.check(lib.bwmoe_combine_peers(peer["y_ptrs"], G, pos.data_ptr(), indices.data_ptr(),
                                               weights.data_ptr(), delta.data_ptr(), el, T, D, K, out.data_ptr(), st))
        self._mark("combine")
        self.last_status = status
        return self._finish(out, host_in)

    def _forward_peers(self, x, weights, indices, row_amax, host_in):
        """Per-tensor recipe over peer memory: route/plan locally, exchange counts and maxima, then
        barrier - quantise-and-store to the owners - barrier - local GEMMs - barrier - combine from the owners."""
        lib, dev, E, K, D, H, el = _lib.lib(), self.dev, self.E, self.K, self.D, self.H, self.el
        G, rank, T = self.world, self.rank, x.shape[0]
        M = T * K
        st = torch.cuda.current_stream(dev).cuda_stream
        i32, f32, u8 = torch.int32, torch.float32, torch.uint8
        new = lambda *shape, dtype: torch.empty(shape, dtype=dtype, device=dev)      # noqa: E731
        peer = self._peer
        if self.profile:
            self._marks = []
        self._mark("start")
        status = torch.zeros(4, dtype=i32, device=dev)
        offsets, pos, row_slot, row_expert = new(E + 1, dtype=i32), new(M, dtype=i32), new(M, dtype=i32), new(M, dtype=i32)
        stats = new(2 * E, dtype=f32)                                   # [amax | counts]
        scratch = new(lib.bwmoe_plan_scratch_bytes(T, E, K), dtype=u8)
        _lib.check(lib.bwmoe_permute_plan(indices.data_ptr(), row_amax.data_ptr(), T, E, K, offsets.data_ptr(),
                                          pos.data_ptr(), row_slot.data_ptr(), row_expert.data_ptr(),
                                          stats[:E].data_ptr(), status.data_ptr(), scratch.data_ptr(), st))
        stats[E:].view(i32).copy_(offsets[1:] - offsets[:-1])
        self._mark("plan")
        gathered = new(G * 2 * E, dtype=f32)
        dist.all_gather_into_tensor(gathered, stats, group=self.group)
        gathered = gathered.view(G, 2 * E)
        amax = gathered[:, :E].amax(0).contiguous()
        counts = gathered[:, E:].contiguous().view(i32)                 # [G, E] rows rank s has for expert e
        self.last_counts = counts
        scale_x = new(E, dtype=f32)
        _lib.check(lib.bwmoe_segment_scales(amax.data_ptr(), None, E, scale_x.data_ptr(), st))
        sx_local = scale_x[rank * el:(rank + 1) * el].contiguous()
        delta, offsets_l, home_counts, home_first = self._peer_maps(counts, offsets)
        # No host synchronisation: the number of rows this rank receives stays on the device.  The GEMMs and the
        # requantisation take their rows from the device-side segment offsets; the buffers are sized for the
        # agreed worst case, and a row beyond it is dropped by the store kernel (status bit).
        cap = peer["cap"]
        self._mark("counts+maps")

        peer["hx"].barrier()             # every rank is done with the previous step's buffers
        self._mark("barrier A")
        _lib.check(lib.bwmoe_scatter_quant_peers(x.data_ptr(), pos.data_ptr(), indices.data_ptr(), scale_x.data_ptr(),
                                                 delta.data_ptr(), T, D, K, el, peer["xq_ptrs"], G, cap,
                                                 status.data_ptr(), st))
        self._mark("quantise+store")
        peer["hx"].barrier()             # every row of this step has landed
        self._mark("barrier B")
        if "h" not in peer:
            peer["h"], peer["hq"] = new(cap, H, dtype=torch.bfloat16), new(cap, H, dtype=u8)
            peer["gs"] = new(max(256, lib.bwmoe_gemm_scratch_bytes(cap, D, H, el)), dtype=u8)
        h, hq, gs = peer["h"], peer["hq"], peer["gs"]
        amax_h = torch.zeros(el, dtype=f32, device=dev)
        _lib.check(lib.bwmoe_gateup_swiglu(peer["xq"].data_ptr(), offsets_l.data_ptr(), sx_local.data_ptr(),
                                           self.wg.data_ptr(), self.wu.data_ptr(), self.sg.data_ptr(),
                                           self.su.data_ptr(), cap, D, H, el, h.data_ptr(), amax_h.data_ptr(),
                                           status.data_ptr(), gs.data_ptr(), st))
        scale_h = new(el, dtype=f32)
        _lib.check(lib.bwmoe_segment_scales(amax_h.data_ptr(), None, el, scale_h.data_ptr(), st))
        _lib.check(lib.bwmoe_requant_segments(h.data_ptr(), offsets_l.data_ptr(), scale_h.data_ptr(), el, H,
                                              hq.data_ptr(), st))
        if self._push():
            _lib.check(lib.bwmoe_down_peers(hq.data_ptr(), offsets_l.data_ptr(), scale_h.data_ptr(),
                                            self.wd.data_ptr(), self.sd.data_ptr(), cap, D, H, el,
                                            home_counts.data_ptr(), home_first.data_ptr(), peer["y_ptrs"], G,
                                            status.data_ptr(), st))
        else:
            _lib.check(lib.bwmoe_down(hq.data_ptr(), offsets_l.data_ptr(), scale_h.data_ptr(), self.wd.data_ptr(),
                                      self.sd.data_ptr(), cap, D, H, el, peer["y"].data_ptr(), status.data_ptr(),
                                      gs.data_ptr(), st))
        self._mark("gate/up+requant+down")
        peer["hy"].barrier()             # every rank's result rows are complete (and, pushed, at home)
        self._mark("barrier C")
        out = new(T, D, dtype=torch.bfloat16)
        if self._push():
            _lib.check(lib.bwmoe_combine(peer["y"].data_ptr(), pos.data_ptr(), weights.data_ptr(), T, D, K,
                                         out.data_ptr(), st))
        else:
            _lib.check(lib.bwmoe_combine_peers(peer["y_ptrs"], G, pos.data_ptr(), indices.data_ptr(),
                                               weights.data_ptr(), delta.data_ptr(), el, T, D, K, out.data_ptr(), st))
        self._mark("combine")
        self.last_status = status
        return self._finish(out, host_in)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        host_in = not x.is_cuda
        if host_in:
            x = x.to(self.dev, non_blocking=True)
        lib, dev, E, K, D, H, el = _lib.lib(), self.dev, self.E, self.K, self.D, self.H, self.el
        T = x.shape[0]
        st = torch.cuda.current_stream(dev).cuda_stream
        i32, f32, u8 = torch.int32, torch.float32, torch.uint8
        new = lambda *shape, dtype: torch.empty(shape, dtype=dtype, device=dev)      # noqa: E731
        weights, indices, row_amax = new(T, K, dtype=f32), new(T, K, dtype=i32), new(T, dtype=f32)
        # routed by the kernel the concatenated batch of all ranks would get on one GPU (equal batches per rank
        # assumed for the size), so that the routing weights, and with them the output, equal the single-GPU ones
        t_as = self.world * T
        need = lib.bwmoe_router_scratch_bytes_as(T, D, E, K, t_as)
        rs = new(need, dtype=u8) if need else None
        _lib.check(lib.bwmoe_router_as(x.data_ptr(), self.w_gate.data_ptr(), T, D, E, K, t_as, weights.data_ptr(),
                                       indices.data_ptr(), row_amax.data_ptr(), rs.data_ptr() if need else None,
                                       need, st))
        peers = self._use_peers(T)
        if self.block:
            if peers:
                return self._forward_block_peers(x, weights, indices, host_in)
            M = T * K
            offsets, pos, row_slot, row_expert = (new(E + 1, dtype=i32), new(M, dtype=i32), new(M, dtype=i32),
                                                  new(M, dtype=i32))
            return self._forward_block(x, weights, indices, offsets, pos, row_slot, row_expert, host_in)
        if peers:
            return self._forward_peers(x, weights, indices, row_amax, host_in)

        # ---- plan every micro-batch, exchange counts and activation maxima once ----
        nmb = self.micro_batches if T >= self.micro_batch_min_tokens * self.micro_batches else 1
        bounds = [T * i // nmb for i in range(nmb + 1)]
        status = torch.zeros(4, dtype=i32, device=dev)
        stats = torch.zeros((1 + nmb) * E, dtype=f32, device=dev)      # [amax | counts of batch 0 | batch 1 ...]
        mbs = []
        for h in range(nmb):
            t0, t1 = bounds[h], bounds[h + 1]
            Th = t1 - t0
            Mh = Th * K
            mb = dict(t0=t0, t1=t1, T=Th, M=Mh, offsets=new(E + 1, dtype=i32), pos=new(Mh, dtype=i32),
                      row_slot=new(Mh, dtype=i32), row_expert=new(Mh, dtype=i32), amax=new(E, dtype=f32))
            scratch = new(lib.bwmoe_plan_scratch_bytes(Th, E, K), dtype=u8)
            _lib.check(lib.bwmoe_permute_plan(indices[t0:t1].data_ptr(), row_amax[t0:t1].data_ptr(), Th, E, K,
                                              mb["offsets"].data_ptr(), mb["pos"].data_ptr(),
                                              mb["row_slot"].data_ptr(), mb["row_expert"].data_ptr(),
                                              mb["amax"].data_ptr(), status.data_ptr(), scratch.data_ptr(), st))
            torch.maximum(stats[:E], mb["amax"], out=stats[:E])
            stats[(1 + h) * E:(2 + h) * E].view(i32).copy_(mb["offsets"][1:] - mb["offsets"][:-1])
            mbs.append(mb)
        gathered = new(self.world * (1 + nmb) * E, dtype=f32)
        dist.all_gather_into_tensor(gathered, stats, group=self.group)
        gathered = gathered.view(self.world, (1 + nmb) * E)
        amax = gathered[:, :E].amax(0).contiguous()                # exact: a max of the same floats
        counts_all = gathered[:, E:].contiguous().view(i32)        # [G, nmb * E]
        counts_host = counts_all.cpu()                             # one synchronisation for every micro-batch
        scale_x = new(E, dtype=f32)
        _lib.check(lib.bwmoe_segment_scales(amax.data_ptr(), None, E, scale_x.data_ptr(), st))
        sx_local = scale_x[self.rank * el:(self.rank + 1) * el].contiguous()

        if nmb > 1:
            _lib.check(lib.bwmoe_set_sm_reserve(self.sm_reserve))
        # ---- quantise and dispatch (asynchronously) ----
        for h, mb in enumerate(mbs):
            mb["plan"] = ExchangePlan(counts_all[:, h * E:(h + 1) * E], self.rank, counts_host[:, h * E:(h + 1) * E])
            xq = new(mb["M"], D, dtype=u8)
            _lib.check(lib.bwmoe_gather_quant(x[mb["t0"]:mb["t1"]].data_ptr(), mb["row_slot"].data_ptr(),
                                              mb["row_expert"].data_ptr(), scale_x.data_ptr(), mb["M"], D, K,
                                              xq.data_ptr(), st))
            mb["recv"], mb["work"] = dispatch_start(xq, mb["plan"], self.group)
        # ---- gate/up as the batches arrive; the segment amax of h spans all batches ----
        amax_h = torch.zeros(el, dtype=f32, device=dev)
        for mb in mbs:
            mb["work"].wait()
            R = mb["plan"].rows_local
            mb["xq_local"] = dispatch_finish(mb["recv"], mb["plan"])
            mb["h"] = new(R, H, dtype=torch.bfloat16)
            if R > 0:
                mb["gs"] = new(max(256, lib.bwmoe_gemm_scratch_bytes(R, D, H, el)), dtype=u8)
                _lib.check(lib.bwmoe_gateup_swiglu(mb["xq_local"].data_ptr(), mb["plan"].offsets.data_ptr(),
                                                   sx_local.data_ptr(), self.wg.data_ptr(), self.wu.data_ptr(),
                                                   self.sg.data_ptr(), self.su.data_ptr(), R, D, H, el,
                                                   mb["h"].data_ptr(), amax_h.data_ptr(), status.data_ptr(),
                                                   mb["gs"].data_ptr(), st))
        scale_h = new(el, dtype=f32)
        _lib.check(lib.bwmoe_segment_scales(amax_h.data_ptr(), None, el, scale_h.data_ptr(), st))
        # ---- requant + down per batch; rows travel home while the next batch computes ----
        for mb in mbs:
            R = mb["plan"].rows_local
            y_local = new(R, D, dtype=torch.bfloat16)
            if R > 0:
                hq = new(R, H, dtype=u8)
                _lib.check(lib.bwmoe_requant(mb["h"].data_ptr(), mb["plan"].row_expert.data_ptr(), scale_h.data_ptr(),
                                             R, H, hq.data_ptr(), st))
                _lib.check(lib.bwmoe_down(hq.data_ptr(), mb["plan"].offsets.data_ptr(), scale_h.data_ptr(),
                                          self.wd.data_ptr(), self.sd.data_ptr(), R, D, H, el, y_local.data_ptr(),
                                          status.data_ptr(), mb["gs"].data_ptr(), st))
            mb["home"], mb["work"] = combine_back_start(y_local, mb["plan"], mb["M"], self.group)
        if nmb > 1:
            _lib.check(lib.bwmoe_set_sm_reserve(0))
        out = new(T, D, dtype=torch.bfloat16)
        for mb in mbs:
            mb["work"].wait()
            _lib.check(lib.bwmoe_combine(mb["home"].data_ptr(), mb["pos"].data_ptr(),
                                         weights[mb["t0"]:mb["t1"]].data_ptr(), mb["T"], D, K,
                                         out[mb["t0"]:mb["t1"]].data_ptr(), st))
        self.last_status = status
        return self._finish(out, host_in)

    def pipeline(self, max_tokens: int, depth: int = 2) -> "ExpertParallelPipeline":
        """Streaming interface for activations in (pinned) host memory; see :class:`ExpertParallelPipeline`."""
        return ExpertParallelPipeline(self, max_tokens, depth)

    def _finish(self, out, host_in):
        if host_in:
            host = torch.empty(out.shape, dtype=out.dtype, pin_memory=True)
            host.copy_(out, non_blocking=True)
            torch.cuda.current_stream(self.dev).synchronize()
            return host
        return out

    def _forward_block(self, x, weights, indices, offsets, pos, row_slot, row_expert, host_in):
        """Block-scale recipe: activation scales are per token, so only row counts are exchanged."""
        lib, dev, E, K, D, H, el = _lib.lib(), self.dev, self.E, self.K, self.D, self.H, self.el
        T = x.shape[0]
        M = T * K
        st = torch.cuda.current_stream(dev).cuda_stream
        i32, f32 = torch.int32, torch.float32
        new = lambda *shape, dtype: torch.empty(shape, dtype=dtype, device=dev)      # noqa: E731
        status = torch.zeros(4, dtype=i32, device=dev)
        scratch = new(lib.bwmoe_plan_scratch_bytes(T, E, K), dtype=torch.uint8)
        _lib.check(lib.bwmoe_permute_plan(indices.data_ptr(), None, T, E, K, offsets.data_ptr(), pos.data_ptr(),
                                          row_slot.data_ptr(), row_expert.data_ptr(), None, status.data_ptr(),
                                          scratch.data_ptr(), st))
        counts = new(self.world * E, dtype=i32)
        dist.all_gather_into_tensor(counts, (offsets[1:] - offsets[:-1]).contiguous(), group=self.group)
        nd, nh = (D + 127) // 128, (H + 127) // 128
        xq, x_inv = new(M, D, dtype=torch.uint8), new(M, nd, dtype=f32)
        _lib.check(lib.bwmoe_gather_quant_group(x.data_ptr(), row_slot.data_ptr(), M, D, K, xq.data_ptr(),
                                                x_inv.data_ptr(), st))
        plan = ExchangePlan(counts.view(self.world, E), self.rank)
        xq_local = dispatch(xq, plan, self.group)
        xinv_local = dispatch(x_inv, plan, self.group)
        R = plan.rows_local
        y_local = new(R, D, dtype=torch.bfloat16)
        if R > 0:
            hq, h_inv = new(R, H, dtype=torch.uint8), new(R, nh, dtype=f32)
            _lib.check(lib.bwmoe_gateup_swiglu_block(xq_local.data_ptr(), xinv_local.data_ptr(), plan.offsets.data_ptr(),
                                                     self.wg.data_ptr(), self.wu.data_ptr(), self.sg.data_ptr(),
                                                     self.su.data_ptr(), R, D, H, el, hq.data_ptr(), h_inv.data_ptr(),
                                                     status.data_ptr(), st))
            _lib.check(lib.bwmoe_down_block(hq.data_ptr(), h_inv.data_ptr(), plan.offsets.data_ptr(), self.wd.data_ptr(),
                                            self.sd.data_ptr(), R, D, H, el, y_local.data_ptr(), status.data_ptr(), st))
        y_home = combine_back(y_local, plan, M, self.group)
        out = new(T, D, dtype=torch.bfloat16)
        _lib.check(lib.bwmoe_combine(y_home.data_ptr(), pos.data_ptr(), weights.data_ptr(), T, D, K, out.data_ptr(), st))
        self.last_status = status
        return self._finish(out, host_in)


class ExpertParallelPipeline:
    """Expert-parallel forward for callers whose activations live in (pinned) host memory: the host->device copy
    of batch i+1 and the device->host copy of batch i-1 run on their own streams beside the compute (and the
    exchange) of batch i.  Every rank must submit the same number of batches in the same order (each forward is
    a collective); numerically a batch is :meth:`ExpertParallelMoE.forward` of that batch.

        pipe = ep.pipeline(max_tokens=16384)
        t0 = pipe.submit(x0)          # returns without waiting for the GPU where the transport allows it
        t1 = pipe.submit(x1)
        y0 = pipe.result(t0)          # pinned host tensor, valid until its slot is reused
    """

    def __init__(self, ep: ExpertParallelMoE, max_tokens: int, depth: int = 2):
        self.ep, self.Tmax, self.depth, self.dev = ep, max_tokens, depth, ep.dev
        if ep.max_tokens_per_rank is None:
            ep.max_tokens_per_rank = max_tokens
        with torch.cuda.device(self.dev):
            self.s_in, self.s_cmp, self.s_out = (torch.cuda.Stream(self.dev) for _ in range(3))
            self.slots = [dict(x=torch.empty(max_tokens, ep.D, dtype=torch.bfloat16, device=self.dev),
                               host=torch.empty(max_tokens, ep.D, dtype=torch.bfloat16, pin_memory=True), y=None,
                               in_done=torch.cuda.Event(), cmp_done=torch.cuda.Event(), out_done=torch.cuda.Event(), T=0)
                          for _ in range(depth)]
        self.ticket = 0

    def submit(self, x_host: torch.Tensor) -> int:
        assert not x_host.is_cuda and x_host.dtype == torch.bfloat16 and x_host.shape[1] == self.ep.D
        T = x_host.shape[0]
        assert 0 < T <= self.Tmax
        slot = self.slots[self.ticket % self.depth]
        first_use = self.ticket < self.depth
        with torch.cuda.device(self.dev):
            if not first_use:
                self.s_in.wait_event(slot["cmp_done"])        # the previous batch in this slot has been consumed
            with torch.cuda.stream(self.s_in):
                slot["x"][:T].copy_(x_host, non_blocking=True)
                slot["in_done"].record(self.s_in)
            self.s_cmp.wait_event(slot["in_done"])
            if not first_use:
                self.s_cmp.wait_event(slot["out_done"])       # its previous result has left the device
            with torch.cuda.stream(self.s_cmp):
                slot["y"] = self.ep.forward(slot["x"][:T])
                slot["cmp_done"].record(self.s_cmp)
            self.s_out.wait_event(slot["cmp_done"])
            with torch.cuda.stream(self.s_out):
                slot["host"][:T].copy_(slot["y"], non_blocking=True)
                slot["out_done"].record(self.s_out)
        slot["T"] = T
        self.ticket += 1
        return self.ticket - 1

    def result(self, ticket: int) -> torch.Tensor:
        assert self.ticket - self.depth <= ticket < self.ticket, "result no longer (or not yet) available"
        slot = self.slots[ticket % self.depth]
        slot["out_done"].synchronize()
        return slot["host"][:slot["T"]]
