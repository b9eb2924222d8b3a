"""Which kernel serves which call. The float32 engine uses the plain kernels throughout; the
bfloat16 engine swaps in the fast ones where their size limits are met and says no otherwise,
in which case the caller falls back to the plain kernel of the same math (never to a CPU or
library path)."""
from __future__ import annotations

import torch

from ..kernels import ops


class KernelPlan:
    MIN_COUNTERS = 4096            # counters allocated at least; more than any one-token step of 64 lanes needs
    SIGMOID_TC_FROM = 17           # sigmoid-weight attention: pieces this long go to the tcgen05 kernel (tiles of 128
                                   # query rows of ONE head), shorter ones to the kernel whose rows are (token, head) pairs

    def __init__(self, engine):
        self.engine = engine
        self.bf16 = engine.dtype == torch.bfloat16
        self._counters = None          # zeroed once; the decode attention kernel leaves them zero
        self._retired = []             # outgrown counter tensors that captured steps may still point to
        self.decode_attention = engine.decode_attention      # "auto", or "split": always the CUDA-core kernel

    def _decode_counters(self, need: int, device) -> torch.Tensor:
        """Zeroed counters for the merge of a decode attention launch. A captured step keeps the address
        it was captured with, so a tensor that has been handed out is never freed: when a later step needs
        more, the smaller tensor stays alive beside the new one."""
        if self._counters is None or self._counters.numel() < need:
            if self._counters is not None:
                self._retired.append(self._counters)
            self._counters = torch.zeros(max(need, self.MIN_COUNTERS), dtype=torch.int32, device=device)
        return self._counters

    @staticmethod
    def decode_run_length(n_seqs: int, head_dim: int, dtype) -> int:
        """Keys per block of the split-KV kernel: one cache page; the reference uses runs of 256
        (src/flash_decode.py:271-272). Depends only on the step's shape, never on its data."""
        return ops.attention_decode_run_len(n_seqs, head_dim, dtype)

    def attention_with_rope(self, ctx, qkv, table, kv, out, n_q, n_kv, head_dim, options, write_kv) -> bool:
        """One-token steps whose projections were not made by the fused norm + QKV kernel (more than 8 rows):
        rotation of q and k and the cache write happen inside the attention kernel, where a kernel for this
        size exists. Returns False (and does nothing) otherwise; the caller then rotates and stores first."""
        if not write_kv:
            return False       # a borrowed cache already holds the owner's new key: it must be read, not replaced
        if not (ctx.decode and self.decode_attention != "split" and qkv.dtype == torch.bfloat16
                and table is not None and ops.attention_decode_mma_supported(head_dim, qkv.dtype, kv.page_size)):
            return False
        pages = ops.attention_decode_mma_pages(ctx.n_seqs, n_q, n_kv, ctx.max_kv_len)
        n_runs = ((ctx.max_kv_len + 63) // 64 + pages - 1) // pages
        counters = self._decode_counters(ops.decode_counter_ints(ctx.n_seqs, n_q, n_kv), qkv.device)
        ops.attention_decode_mma_rope(qkv, kv.k, kv.v, out, table, ctx.seq_slot, ctx.seq_kvlen, kv.block_table,
                                      kv.page_size, n_q, n_kv, head_dim, options.scale, options.window, pages, n_runs,
                                      write_kv, counters=counters)
        return True

    def attention(self, ctx, q, kv, out, n_q, n_kv, head_dim, options, gate=None) -> bool:
        """Returns True when a specialised kernel ran (the gate, if any, applied). The tensor-core kernels know
        every option (scale, window, kept first keys, sink, gate); the CUDA-core split-KV kernel knows scale and
        window. A value head size that differs from the key head size is the plain kernel's alone."""
        scale, window = options.scale, options.window
        if options.sigmoid_bias is not None:
            return self._sigmoid_attention(ctx, q, kv, out, n_q, n_kv, head_dim, options, gate)
        if kv.v.shape[-1] != head_dim or not kv.v.is_contiguous():
            # a value size of its own, or values that are columns of the key rows (a latent)
            return self._attention_by_rows(ctx, q, kv, out, n_q, n_kv, head_dim, options, gate)
        if gate is not None and (gate.stride(0) % 8 or gate.data_ptr() % 16):
            # the tensor-core kernels load the gate 16 bytes at a time: rows that do not start on 16 bytes are
            # applied by a kernel of their own afterwards
            if not self.attention(ctx, q, kv, out, n_q, n_kv, head_dim, options, None):
                return False
            ops.sigmoid_gate(out, gate)
            return True
        if ctx.decode and self.decode_attention != "split" \
                and ops.attention_decode_mma_supported(head_dim, q.dtype, kv.page_size):
            # bfloat16, head size 64 or 128: a warp per page on the tensor cores
            pages = ops.attention_decode_mma_pages(ctx.n_seqs, n_q, n_kv, ctx.max_kv_len)
            n_runs = ((ctx.max_kv_len + 63) // 64 + pages - 1) // pages
            counters = self._decode_counters(ops.decode_counter_ints(ctx.n_seqs, n_q, n_kv), q.device)
            ops.attention_decode_mma(q, kv.k, kv.v, out, ctx.seq_slot, ctx.seq_kvlen, kv.block_table, kv.page_size,
                                     n_q, n_kv, head_dim, scale, window, pages, n_runs, counters=counters,
                                     keep_first=options.keep_first, sink=options.sink, gate=gate,
                                     softcap=options.softcap, dist_bias=options.distance_bias,
                                     sink_values=options.sink_values)
            return True
        if not ctx.decode and scale > 0 and ops.attention_prefill_tc_supported(head_dim, kv.page_size, q.dtype):
            ops.attention_prefill_tc(q, kv.k, kv.v, out, ctx.cu_q, ctx.seq_slot, ctx.seq_start, kv.block_table,
                                     kv.page_size, ctx.n_seqs, ctx.max_q_len, n_q, n_kv, head_dim, scale, window,
                                     options.keep_first, options.sink, gate, options.softcap, options.distance_bias,
                                     options.sink_values)
            return True
        if options.scored:
            # a cap, a bias by distance or a learned sink: the split-KV kernel below does not know them
            return self._attention_by_rows(ctx, q, kv, out, n_q, n_kv, head_dim, options, gate)
        if ctx.decode and options.plain and kv.page_size == 64 and ops.attention_decode_supported(head_dim, q.dtype):
            run = self.decode_run_length(ctx.n_seqs, head_dim, q.dtype)
            n_runs = (ctx.max_kv_len + run - 1) // run
            counters = self._decode_counters(ops.decode_counter_ints(ctx.n_seqs, n_q, n_kv), q.device)
            ops.attention_decode(q, kv.k, kv.v, out, ctx.seq_slot, ctx.seq_kvlen, kv.block_table, kv.page_size,
                                 n_q, n_kv, head_dim, scale, window, run, n_runs, counters=counters)
            if gate is not None:
                ops.sigmoid_gate(out, gate)
            return True
        return False

    def _sigmoid_attention(self, ctx, q, kv, out, n_q, n_kv, head_dim, options, gate) -> bool:
        """Attention without a softmax (weights sigmoid(score + a number per head), not normalised). Prompts of the
        bfloat16 engine with head size 64 or 128 (values of the same size): the tcgen05 kernel; their one-token steps:
        the kernel with a warp per cache page. Other sizes and short pieces: the tensor-core kernel by rows. What that does not take (float32, head sizes that are no
        multiples of 16) is the plain kernel's."""
        square = kv.v.shape[-1] == head_dim and kv.v.is_contiguous()
        aligned_gate = gate is None or not (gate.stride(0) % 8 or gate.data_ptr() % 16)
        if not ctx.decode and ctx.max_q_len >= self.SIGMOID_TC_FROM and options.scale > 0 and square and aligned_gate \
                and ops.attention_prefill_tc_supported(head_dim, kv.page_size, q.dtype):
            ops.attention_prefill_tc(q, kv.k, kv.v, out, ctx.cu_q, ctx.seq_slot, ctx.seq_start, kv.block_table,
                                     kv.page_size, ctx.n_seqs, ctx.max_q_len, n_q, n_kv, head_dim, options.scale,
                                     options.window, options.keep_first, False, gate,
                                     sigmoid_bias=options.sigmoid_bias)
            return True
        if ctx.decode and self.decode_attention != "split" and square and aligned_gate \
                and ops.attention_decode_mma_supported(head_dim, q.dtype, kv.page_size):
            pages = ops.attention_decode_mma_pages(ctx.n_seqs, n_q, n_kv, ctx.max_kv_len)
            n_runs = ((ctx.max_kv_len + 63) // 64 + pages - 1) // pages
            counters = self._decode_counters(ops.decode_counter_ints(ctx.n_seqs, n_q, n_kv), q.device)
            ops.attention_decode_mma(q, kv.k, kv.v, out, ctx.seq_slot, ctx.seq_kvlen, kv.block_table, kv.page_size,
                                     n_q, n_kv, head_dim, options.scale, options.window, pages, n_runs,
                                     counters=counters, keep_first=options.keep_first, gate=gate,
                                     sigmoid_bias=options.sigmoid_bias)
            return True
        return self._attention_by_rows(ctx, q, kv, out, n_q, n_kv, head_dim, options, gate)

    def _attention_by_rows(self, ctx, q, kv, out, n_q, n_kv, head_dim, options, gate) -> bool:
        """The tensor-core kernel whose rows are the (token, head) pairs of a key/value head: prompts and one-token
        steps of the shapes and options the kernels above do not take. It knows no kept first keys."""
        shared_rows = not kv.v.is_contiguous()
        if options.keep_first or not ops.attention_rows_mma_supported(head_dim, kv.v.shape[-1], kv.page_size, q.dtype,
                                                                      shared_rows):
            return False
        ops.attention_rows_mma(q, kv.k, kv.v, out, ctx.cu_q, ctx.seq_slot, ctx.seq_start, kv.block_table, kv.page_size,
                               ctx.n_seqs, ctx.max_q_len, n_q, n_kv, head_dim, options.scale, options.window,
                               options.softcap, options.distance_bias, options.sink_values, options.sink,
                               options.sigmoid_bias)
        if gate is not None:
            ops.sigmoid_gate(out, gate)
        return True
