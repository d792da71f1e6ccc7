# SPDX-License-Identifier: MIT
"""Communicator used by the tensor-parallel layers.

On CUDA with the link up, every call is one hand-written kernel of the link
core (`_C.allreduce_into`, `_C.allreduce_rmsnorm`, `_C.allgather_into`): no
c10d dispatch on the hot path.  On CPU (or with a foreign backend such as
gloo / nccl for A/B runs) the same calls go through `torch.distributed`.
The reference's equivalent is the `dist.all_reduce` forward hook on
row-parallel modules (demos/qwen_tp/qwen38_int8/worker.py:167-183) and the
isend/irecv lm_head exchange (:223-241).
"""
import torch
import torch.distributed as dist

from .. import load_extension
from ..ops import reference as ref
from .. import ops as _ops


# BL_PUSH_AR when the environment does not set it ("1": row-parallel linears of 129 rows or more
# scatter their tiles themselves, see TPComm.row_parallel)
PUSH_AR_DEFAULT = "0"


class TPComm:
    def __init__(self, group=None, use_link=None):
        if group is None and dist.is_available() and dist.is_initialized():
            group = dist.group.WORLD
        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        if use_link is None:
            use_link = False
            if self.world > 1 and torch.cuda.is_available():
                try:
                    info = load_extension().info()
                    use_link = bool(info.get("initialized") and info.get("peer_mode")
                                    and info.get("world") == self.world)
                except ImportError:
                    use_link = False
        self.use_link = use_link
        self.oneshot_max = load_extension().info()["oneshot_max"] if use_link else 0
        self.max_chunk = load_extension().info()["max_chunk"] if use_link else 0
        self.ar_calls = 0
        self.ar_bytes = 0
        # timing control of the reference's demos (`--no-comm`,
        # demos/qwen_tp/qwen38_int8/worker.py:157-183): every collective is
        # skipped, results are wrong, the step time is compute only
        self.no_comm = False
        self._init_timing()

    def _init_timing(self):
        # per-collective device timing (the reference brackets every hooked all_reduce with CUDA
        # events and reports their sum, demos/qwen_tp/qwen38_int8/worker.py:157-183, 630-637):
        # eager steps only, never while a stream is being captured
        self.time_collectives = False
        self._timed = []

    def _timed_call(self, fn):
        if not self.time_collectives or not torch.cuda.is_available() or torch.cuda.is_current_stream_capturing():
            return fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        r = fn()
        b.record()
        self._timed.append((a, b))
        return r

    def collective_ms(self, reset=True):
        """(calls, total device ms) of the collectives timed since the last reset."""
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        n, ms = len(self._timed), sum(a.elapsed_time(b) for a, b in self._timed)
        if reset:
            self._timed = []
        return n, ms

    @classmethod
    def single(cls):
        """A communicator of one rank: every collective is a local no-op."""
        c = cls.__new__(cls)
        c.group, c.world, c.rank = None, 1, 0
        c.use_link, c.oneshot_max, c.ar_calls, c.ar_bytes, c.max_chunk = False, 0, 0, 0, 0
        c.no_comm = False
        c._init_timing()
        return c

    # ---- collectives -----------------------------------------------------
    def all_reduce(self, x):
        """In-place sum over the group; returns x."""
        if self.world == 1 or self.no_comm:
            return x
        self.ar_calls += 1
        self.ar_bytes += x.numel() * x.element_size()
        if self.use_link and x.is_cuda and x.is_contiguous() and (x.numel() * x.element_size()) % 16 == 0 \
                and x.data_ptr() % 16 == 0:
            nbytes = x.numel() * x.element_size()
            if nbytes <= self.max_chunk:
                _ops._count()
                self._timed_call(lambda: load_extension().allreduce_into(x, x))
            else:
                flat = x.view(-1)
                step = (self.max_chunk // 16 * 16) // x.element_size()
                for i in range(0, flat.numel(), step):
                    _ops._count()
                    part = flat[i:i + step]
                    load_extension().allreduce_into(part, part)
            return x
        self._timed_call(lambda: dist.all_reduce(x, group=self.group))
        return x

    def row_parallel(self, out, parts):
        """out[row0 : row0 + rows] = sum over ranks of (x @ w.T (+ bias) (GELU) (+ residual)) for every
        part (x, w, bias, residual, gelu, row0); the parts tile the rows of out [T, n].

        On the link, for token-major sizes, the GEMM epilogue is the scatter half of a two-shot
        all-reduce: every finished 128 x 256 tile is stored as bf16 straight into the staging inbox
        of the rank that owns those rows (peer stores over NVLink while the other tiles are still
        in the tensor cores) and one more kernel reduces this rank's rows and hands the sums to
        every rank.  BL_PUSH_AR=0, other sizes and other backends: GEMM into out, then all_reduce."""
        import os
        T, n = out.shape
        fused = (self.world > 1 and self.use_link and out.is_cuda and not self.no_comm
                 and out.dtype == torch.bfloat16 and out.is_contiguous()
                 and os.environ.get("BL_PUSH_AR", PUSH_AR_DEFAULT) != "0"
                 and T % self.world == 0 and n >= 256 and n % 8 == 0
                 and (T // self.world) * n * 2 <= self.max_chunk // self.world
                 and all(p[0].shape[0] > 128 and p[0].dtype == torch.bfloat16 for p in parts))
        if fused:
            C = load_extension()
            units = 0
            for x, w, bias, residual, gelu, row0 in parts:
                _ops._count()
                units += C.linear_push(x, w, bias, residual, gelu, T, row0)
            _ops._count()
            self.ar_calls += 1
            self.ar_bytes += out.numel() * out.element_size()
            self._timed_call(lambda: C.allreduce_pushed(out, units))
            return out
        for x, w, bias, residual, gelu, row0 in parts:
            _ops.linear(x, w, bias, residual=residual, gelu=gelu, out=out[row0:row0 + x.shape[0]])
        if self.world > 1:
            self.all_reduce(out)
        return out

    def all_gather_cols(self, x):
        """[rows, n_local] on every rank -> [rows, world * n_local] (rank-major columns)."""
        if self.world == 1:
            return x
        rows, n = x.shape
        flat = torch.empty(self.world, rows, n, dtype=x.dtype, device=x.device)
        xc = x.contiguous()
        if self.use_link and x.is_cuda and (xc.numel() * xc.element_size()) % 16 == 0:
            _ops._count()
            load_extension().allgather_into(flat.view(-1), xc.view(-1))
        else:
            dist.all_gather_into_tensor(flat.view(-1), xc.view(-1), group=self.group)
        return flat.permute(1, 0, 2).reshape(rows, self.world * n)

    def all_gather_rows(self, x):
        """[rows_local, n] -> [world * rows_local, n]."""
        if self.world == 1:
            return x
        xc = x.contiguous()
        out = torch.empty(self.world * xc.shape[0], *xc.shape[1:], dtype=x.dtype, device=x.device)
        if self.use_link and x.is_cuda and (xc.numel() * xc.element_size()) % 16 == 0:
            _ops._count()
            load_extension().allgather_into(out.view(-1), xc.view(-1))
        else:
            dist.all_gather_into_tensor(out.view(-1), xc.view(-1), group=self.group)
        return out

    def allreduce_rmsnorm(self, x, residual, gamma, eps):
        """(normed, new_residual) where new_residual = all_reduce(x) + residual.

        One kernel on the link when the message fits the one-shot inbox;
        otherwise all-reduce followed by the add+norm kernel."""
        if self.world == 1 or self.no_comm:
            if x.dtype == torch.float32 and x.dim() == 3 and gamma.dtype != torch.float32 and not x.is_cuda:
                x = x.sum(0).to(gamma.dtype)
            return _ops.rmsnorm(x, gamma, eps, residual)
        slabs = x.dtype == torch.float32 and x.dim() == 3 and gamma.dtype != torch.float32
        nbytes = (x[0].numel() * gamma.element_size()) if slabs else x.numel() * x.element_size()
        if slabs and not (self.use_link and x.is_cuda and nbytes <= self.oneshot_max):
            x = x.sum(0).to(gamma.dtype)  # no fused path for this size: fold the k-split slabs here
            slabs = False
        if self.use_link and x.is_cuda and nbytes <= self.oneshot_max and x.is_contiguous():
            self.ar_calls += 1
            self.ar_bytes += nbytes
            _ops._count()
            normed, res = self._timed_call(
                lambda: load_extension().allreduce_rmsnorm(x, residual, gamma, eps, None, residual))
            return normed, res
        self.all_reduce(x)
        if residual is None:
            normed, _ = _ops.rmsnorm(x, gamma, eps)
            return normed, x
        return _ops.rmsnorm(x, gamma, eps, residual)

    def argmax_vocab_parallel(self, logits_local, vocab_per_rank, out=None):
        """Global arg max over vocab-parallel logits [rows, vocab_per_rank] (int32 [rows], written
        to `out` when given).  On the link: the arg max kernel leaves (value, index) pairs per slice
        of a row in the layout the merge kernel reads, the pairs of all ranks are all-gathered as
        they are, and one merge kernel picks -- three launches, no repacking in between."""
        if logits_local.is_cuda and self.use_link and self.world > 1 and not self.no_comm:
            C = load_extension()
            parts = C.argmax_parts(logits_local, self.rank * vocab_per_rank)       # [chunks, rows, 2]
            if parts.numel() * 4 % 16 == 0:
                allp = torch.empty(self.world * parts.shape[0], parts.shape[1], 2, dtype=torch.float32,
                                   device=parts.device)
                _ops._count(3)
                C.allgather_into(allp.view(-1), parts.view(-1))
                return C.argmax_merge(allp, out)
        idx, val = _ops.argmax(logits_local, self.rank * vocab_per_rank)
        if self.world == 1 or self.no_comm:
            if out is not None:
                out.copy_(idx)
                return out
            return idx
        pairs = torch.stack([val, idx.view(torch.float32) if idx.dtype == torch.int32 else idx.float()], -1)
        if logits_local.is_cuda and self.use_link:
            rows = pairs.shape[0]
            pad = (-rows) % 2  # 8 bytes per row: pad to a 16-byte multiple
            if pad:
                pairs = torch.cat([pairs, pairs.new_zeros(pad, 2)], 0)
            allp = torch.empty(self.world, rows + pad, 2, dtype=torch.float32, device=pairs.device)
            _ops._count(2)
            load_extension().allgather_into(allp.view(-1), pairs.contiguous().view(-1))
            r = load_extension().argmax_merge(allp[:, :rows].contiguous())
            if out is not None:
                out.copy_(r)
                return out
            return r
        vals = [torch.empty_like(val) for _ in range(self.world)]
        idxs = [torch.empty_like(idx) for _ in range(self.world)]
        dist.all_gather(vals, val.contiguous(), group=self.group)
        dist.all_gather(idxs, idx.contiguous(), group=self.group)
        v = torch.stack(vals, 0)
        i = torch.stack(idxs, 0)
        # highest value, lowest index on ties
        best = v.max(0).values
        cand = torch.where(v == best[None], i, torch.full_like(i, 2 ** 31 - 1))
        r = cand.min(0).values.to(torch.int32)
        if out is not None:
            out.copy_(r)
            return out
        return r

    def barrier(self):
        if self.world > 1:
            dist.barrier(group=self.group)
