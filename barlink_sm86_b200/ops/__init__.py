# SPDX-License-Identifier: MIT
"""Op surface used by the models.

CUDA tensors always run the sm_100a kernels of the compiled extension (and
fail loudly when it is missing); CPU tensors run the fp32 PyTorch statements
in `reference.py`, which are also the oracles of the GPU tests.  The
reference's op surface is `w8a16_quant_act` / `w8a16_gemm`
(torch_ext/barlink_sm86/binding.cpp:434-490); everything else here replaces
library or eager-framework kernels that its demos call.
"""
import torch

from .. import load_extension
from . import reference as ref

# number of sm_100a kernel launches issued through this module (bench.py reports it)
launch_count = 0


def _C():
    return load_extension()


def _count(n=1):
    global launch_count
    launch_count += n


class TiledWeight:
    """A linear layer's weight [n, k] stored as 16 KiB tiles in the layout the
    tensor core reads from shared memory, so that the GEMM fetches a tile with
    one bulk copy.  Built once at load with `tile_weight`."""

    __slots__ = ("data", "n", "k")

    def __init__(self, data, n, k):
        self.data, self.n, self.k = data, n, k

    @property
    def shape(self):
        return (self.n, self.k)

    def numel(self):
        return self.data.numel()

    def element_size(self):
        return self.data.element_size()


def tile_weight(weight):
    """[n, k] bf16 CUDA tensor -> TiledWeight (other tensors are returned as is)."""
    if isinstance(weight, TiledWeight) or not weight.is_cuda or weight.dtype != torch.bfloat16:
        return weight
    n, k = weight.shape
    return TiledWeight(_C().tile_weight(weight.contiguous()), n, k)


def untile_weight(weight):
    """TiledWeight -> the plain [n, k] tensor (other tensors are returned as is)."""
    if not isinstance(weight, TiledWeight):
        return weight
    n, k = weight.n, weight.k
    rt, kb = -(-n // 128), -(-k // 64)
    t = weight.data[: rt * kb * 8192].view(rt, kb, 128, 8, 8)
    r = torch.arange(128, device=t.device)[:, None]
    c = torch.arange(8, device=t.device)[None, :]
    phys = (c ^ (r & 7))[None, None, :, :, None].expand(rt, kb, 128, 8, 8)  # 16-byte chunk c of row r sits at c ^ (r & 7)
    return torch.gather(t, 3, phys).permute(0, 2, 1, 3, 4).reshape(rt * 128, kb * 64)[:n, :k].contiguous()


def _w(weight):
    if isinstance(weight, TiledWeight):
        return weight.data, weight.n, weight.k
    return weight, 0, 0


def linear(x, weight, bias=None, residual=None, silu_mul=False, out=None, gate_tokens=0, gelu=False,
           dynamic_weights=False):
    """y = x @ weight.T (+ bias) (tanh-GELU if `gelu`) (+ residual).
    gate_tokens > 0: x is the all-gather buffer of the fused tensor-parallel
    path; the kernel waits for the peers' rows before it reads x.
    dynamic_weights: `weight` was written by a kernel earlier in this stream
    (not at load time), so its tiles must not be fetched ahead of that kernel."""
    if x.is_cuda:
        _count()
        x2 = x if x.dim() == 2 else x.reshape(-1, x.shape[-1])
        w, tn, tk = _w(weight)
        y = _C().linear(x2, w, bias, residual, silu_mul, out, gate_tokens=gate_tokens, tiled_n=tn,
                        tiled_k=tk, gelu=gelu, dynamic_weights=dynamic_weights)
        return y if x.dim() == 2 else y.view(*x.shape[:-1], y.shape[-1])
    y = ref.linear(x, weight, bias, residual, silu_mul, gelu)
    if out is not None:
        out.copy_(y)
        return out
    return y


def k_splits(x, weight):
    """Number of k-splits `linear_split` would use for this call (1: none)."""
    if x.is_cuda and x.dim() == 2 and x.shape[0] <= 128:
        return _C().gemm_splits(weight.shape[0], weight.shape[1], x.shape[0])
    return 1


def linear_split(x, weight, gate_tokens=0):
    """Decode-path linear: when the shape wants a k-split, returns fp32 slabs
    [splits, tokens, n] whose sum is x @ weight.T (the consumer -- `rmsnorm`,
    `rope_kv_write`, the fused all-reduce -- adds them while reading, so the
    GEMM has no reduction tail); otherwise the plain bf16 result."""
    if x.is_cuda and x.dim() == 2 and x.shape[0] <= 128:
        C = _C()
        splits = C.gemm_splits(weight.shape[0], weight.shape[1], x.shape[0])
        if splits > 1:
            _count()
            w, tn, tk = _w(weight)
            return C.linear_partial(x, w, splits, None, gate_tokens, tn, tk)
    return linear(x, weight, gate_tokens=gate_tokens)


def rmsnorm(x, gamma, eps, residual=None, out=None):
    """Returns (normed, residual); the residual tensor is updated in place on CUDA."""
    if x.is_cuda:
        _count()
        return _C().rmsnorm(x, gamma, eps, residual, out)
    return ref.rmsnorm(x, gamma, eps, residual)


def rope_kv_write(qkv, positions, slots, k_cache, v_cache, nq, nkv, hd, block_size, theta, bias=None):
    """qkv: bf16 [rows, width] rotated in place, or fp32 split-K slabs of the
    QKV linear (then `bias` is added and a new bf16 buffer is returned)."""
    if qkv.is_cuda:
        _count()
        return _C().rope_kv_write(qkv, positions, slots, k_cache, v_cache, nq, nkv, hd, block_size,
                                  theta, bias)
    if bias is not None:
        qkv = (qkv.float() + bias.float()).to(qkv.dtype)
    return ref.rope_kv_write(qkv, positions, slots, k_cache, v_cache, nq, nkv, hd, block_size, theta)


def rope(x, positions, theta, axes=1):
    """x [rows, heads, hd]; rotated in place on CUDA."""
    if x.is_cuda:
        _count()
        rows, heads, hd = x.shape
        _C().rope(x.view(rows, heads * hd), positions, heads, hd, theta, axes)
        return x
    return ref.rope(x, positions, theta, axes)


def w4a16_linear(x, qweight, scales, qzeros, group_size=128):
    """Weight-only int4 linear on GPTQ-v1 tensors (see `ref.pack_int4`): a
    hand-written GEMV for 1..16 rows, widen + GEMM above that."""
    if x.is_cuda:
        _count(2)
        x2 = x if x.dim() == 2 else x.reshape(-1, x.shape[-1])
        y = _C().w4a16_linear(x2.contiguous(), qweight, scales, qzeros, group_size)
        return y if x.dim() == 2 else y.view(*x.shape[:-1], y.shape[-1])
    return ref.w4a16_linear(x, qweight, scales, qzeros, group_size)


def qknorm_rope(qkv, gq, gk, positions, heads, eps=1e-6, theta=1e4, axes=2):
    """In place on the first 2*heads*128 columns of qkv [rows, width]: per-head
    RMSNorm of the q and k heads (weights gq, gk; None = no norm), then RoPE
    with `axes` position coordinates per row (positions int32 [rows, axes])."""
    if qkv.is_cuda:
        _count()
        _C().qknorm_rope(qkv, gq, gk, positions, heads, eps, theta, axes)
        return qkv
    return ref.qknorm_rope(qkv, gq, gk, positions, heads, eps, theta, axes)


def layernorm_modulate(x, shift, scale, rows_per_batch, eps=1e-6):
    """LayerNorm(x) * (1 + scale[b]) + shift[b] with b = row // rows_per_batch
    (adaLN modulation; shift/scale are [batch, hidden] views of one row pitch)."""
    if x.is_cuda:
        _count()
        return _C().layernorm_modulate(x, shift, scale, rows_per_batch, eps)
    return ref.layernorm_modulate(x, shift, scale, rows_per_batch, eps)


def gate_residual(x, y, gate, rows_per_batch):
    """x += gate[b] * y in place; returns x."""
    if x.is_cuda:
        _count()
        _C().gate_residual(x, y, gate, rows_per_batch)
        return x
    return ref.gate_residual(x, y, gate, rows_per_batch)


def silu_mul(gate_up, interleaved=False):
    if gate_up.is_cuda:
        _count()
        return _C().silu_mul(gate_up, interleaved)
    return ref.silu_mul(gate_up, interleaved)


def embedding(ids, table, vocab_lo=0, out=None):
    if table.is_cuda:
        _count()
        return _C().embedding(ids, table, vocab_lo, out)
    return ref.embedding(ids, table, vocab_lo)


def argmax(logits, offset=0):
    if logits.is_cuda:
        _count()
        return _C().argmax(logits, offset)
    return ref.argmax(logits, offset)


def paged_attn_decode(qkv, k_cache, v_cache, block_tables, ctx_lens, nq, nkv, hd, scale, splits=0,
                      out=None):
    if qkv.is_cuda:
        _count(2 if splits != 1 else 1)
        return _C().paged_attn_decode(qkv, k_cache, v_cache, block_tables, ctx_lens, nq, nkv, hd,
                                      scale, splits, out)
    return ref.paged_attn_decode(qkv, k_cache, v_cache, block_tables, ctx_lens, nq, nkv, hd, scale)


def rope_attn_decode(qkv, bias, positions, slots, k_cache, v_cache, block_tables, ctx_lens, nq, nkv, hd,
                     block_size, theta, scale, splits=0):
    """Decode step of one layer's attention in one launch: RoPE on q and the
    new k, the new k/v stored at `slots`, paged attention over the context.
    qkv: bf16 [batch, width] or the fp32 k-split slabs of the QKV linear
    (+ bias).  Same result as rope_kv_write followed by paged_attn_decode."""
    if k_cache.is_cuda:
        _count()  # the splits are merged inside the kernel
        return _C().rope_attn_decode(qkv, bias, positions, slots, k_cache, v_cache, block_tables, ctx_lens,
                                     nq, nkv, hd, theta, scale, splits)
    rot = rope_kv_write(qkv, positions, slots, k_cache, v_cache, nq, nkv, hd, block_size, theta, bias)
    return ref.paged_attn_decode(rot, k_cache, v_cache, block_tables, ctx_lens, nq, nkv, hd, scale)


def attention(q, k, v, cu_q, cu_k, max_q, scale, causal, max_k=0):
    """Dense attention over packed sequences (prefill, joint attention).
    With max_k (length of the longest key sequence) the tcgen05 kernel runs
    (V transpose + attention: two launches); without it the mma.sync kernel."""
    if q.is_cuda:
        _count(2 if max_k > 0 else 1)
        return _C().attn_fwd(q, k, v, cu_q, cu_k, max_q, scale, causal, max_k)
    return ref.attention(q, k, v, cu_q, cu_k, scale, causal)


class W8GroupScales:
    """Per-group int8 scales [n, k/group] in the form the W8A16 kernel applies inside its main
    loop: `row` bf16 [n] (each row's largest scale, applied by the epilogue) and `rel` fp16
    [n, groups] (the group scales divided by it, applied while the int8 tile is widened).
    Build once per weight with `prepare_w8_scales`."""
    __slots__ = ("row", "rel", "group")

    def __init__(self, row, rel, group):
        self.row, self.rel, self.group = row, rel, group


def prepare_w8_scales(scale, k):
    """bf16 group scales [n, k/group] on a CUDA device -> W8GroupScales."""
    row, rel = _C().w8_group_scales(scale.contiguous())
    return W8GroupScales(row, rel, k // scale.shape[1])


def w8_act_mode():
    """How `w8a16_linear` treats the activations by default: "bf16" (weights widened to bf16 in the
    kernel, the activations as they are: the accurate form) or "int8" (activations quantised per token,
    int8 x int8 on the tensor cores: the reference kernel's numerics).  Environment BL_W8_ACT."""
    import os
    v = os.environ.get("BL_W8_ACT", "bf16")
    if v not in ("bf16", "int8"):
        raise ValueError("BL_W8_ACT must be bf16 or int8")
    return v


def w8a16_linear(x, wq, scale, bias=None, silu_mul=False, act=None):
    """scale [n]: per output channel.  scale [n, k/group] or a W8GroupScales: per group, the
    reference's granularity (torch_ext/barlink_sm86/w8a16.cu:119-142 applies group scales inside
    its K loop; so does the tcgen05 kernel here, in the warps that widen the int8 tile).  Group
    sizes that are not multiples of 64, and more than 256 tokens, widen the weight once and run
    the bf16 GEMM.

    act="int8" (per-channel scales only): the activations are quantised per token to int8 first,
    as the reference does (w8a16.cu:37-92 there), and the product runs as `tcgen05.mma kind::i8`
    with int32 accumulators: the weights go from HBM to the tensor cores without being widened, for
    any number of tokens; with group scales [n, k/group] (group a multiple of 128, at most 64 tokens)
    every k-block is accumulated on its own and the epilogue warps apply the scales.  act=None takes
    `w8_act_mode()`."""
    if x.is_cuda:
        k = wq.shape[1]
        gs = scale if isinstance(scale, W8GroupScales) else None
        if (act or w8_act_mode()) == "int8" and gs is None and k % 16 == 0:
            if scale.dim() == 1:
                _count(2)
                return _C().w8a16_linear(x, wq, scale, bias, silu_mul, act_int8=True)
            # (no k-split in that form: it pays from one 128-row tile per SM upwards; below, the widening form)
            if x.shape[0] <= 64 and (k // scale.shape[1]) % 128 == 0 and wq.shape[0] >= 148 * 128:
                # group scales (the reference's checkpoint format): one accumulator per k-block,
                # scaled and summed by the epilogue warps
                _count(2)
                return _C().w8a16_linear(x, wq, scale, bias, silu_mul, act_int8=True, group_scale=scale.contiguous())
        if gs is None and scale.dim() == 2:
            if (k // scale.shape[1]) % 64 == 0 and x.shape[0] <= 256:
                _count()
                gs = prepare_w8_scales(scale, k)
            else:
                w = ref.w8_dequant(wq, scale).to(torch.bfloat16)
                return linear(x, w, bias, silu_mul=silu_mul, dynamic_weights=True)
        _count()
        if gs is not None:
            if x.shape[0] > 256:
                w = (ref.w8_dequant(wq, gs.rel.float() * gs.row.float()[:, None])).to(torch.bfloat16)
                return linear(x, w, bias, silu_mul=silu_mul, dynamic_weights=True)
            return _C().w8a16_linear(x, wq, gs.row, bias, silu_mul, group_rel=gs.rel)
        return _C().w8a16_linear(x, wq, scale, bias, silu_mul)
    if isinstance(scale, W8GroupScales):
        scale = scale.rel.float() * scale.row.float()[:, None]
    return ref.w8a16_linear(x, wq, scale, bias, silu_mul)


__all__ = [
    "linear", "linear_split", "k_splits", "TiledWeight", "tile_weight", "untile_weight", "rmsnorm", "rope_kv_write", "rope", "silu_mul", "embedding", "argmax",
    "paged_attn_decode", "rope_attn_decode", "attention", "w8a16_linear", "W8GroupScales", "prepare_w8_scales", "w4a16_linear", "qknorm_rope", "layernorm_modulate", "gate_residual", "ref",
]
