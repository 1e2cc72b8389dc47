"""Tensor-parallel (Megatron-style, sequence-parallel) MLP and attention-output blocks built on the
fused kernels.  Activations between blocks are sharded by tokens (M / ranks rows per rank); weights
are sharded along the hidden FFN dimension.

  MLP:   X_r [M/R, H]  --all-gather->GEMM with SwiGLU in its epilogue-->  act [M, F/R]
                       --GEMM->reduce-scatter-->  Y_r [M/R, H]
  attention output projection:  A [M, H/R]  --GEMM->reduce-scatter-->  Y_r [M/R, H]

The reference has no model or parallelism code; the shapes are those of the tensor-parallel
benchmark configuration (Llama-3-8B: H = 4096, F = 14336, TP = 8, 4096 tokens)."""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F

from ..ops.elementwise import swiglu_bf16
from ..ops.fused import AllGatherGemm, GemmReduceScatter, interleave_gate_up, split_gate_up


class TensorParallelMLP:
    def __init__(self, comm, tokens: int, hidden: int, ffn: int, seed: int = 0, n_comm_ctas: int = 0):
        R = comm.size
        if ffn % R:
            raise ValueError("ffn must divide by the number of ranks")
        self.comm, self.tokens, self.hidden, self.ffn_local = comm, tokens, hidden, ffn // R
        g = torch.Generator(device="cuda").manual_seed(seed * 1000 + comm.rank)
        std = 0.02
        # nn.Linear layout [out_features, in_features].  Gate and up are stored as ONE matrix whose rows are
        # interleaved in groups of 16, the layout the SwiGLU epilogue of the all-gather->GEMM kernel consumes.
        w_gate = (torch.randn(self.ffn_local, hidden, generator=g, device="cuda") * std).to(torch.bfloat16)
        w_up = (torch.randn(self.ffn_local, hidden, generator=g, device="cuda") * std).to(torch.bfloat16)
        if self.ffn_local % 16:
            raise ValueError("ffn / ranks must be a multiple of 16")
        self.w_gate_up = interleave_gate_up(w_gate, w_up)
        self.w_gate_up_plain = torch.cat((w_gate, w_up))  # (gate | up) stacked: what the library-only baseline multiplies by
        self.w_down = (torch.randn(hidden, self.ffn_local, generator=g, device="cuda") * std).to(torch.bfloat16)
        self.ag_gemm = AllGatherGemm(comm, tokens, hidden, n_comm_ctas=n_comm_ctas)
        self.gemm_rs = GemmReduceScatter(comm, tokens, hidden)
        self._act = torch.empty(tokens, self.ffn_local, dtype=torch.bfloat16, device="cuda")
        # MINI_NCCL_TP_SWIGLU=separate keeps the H = (gate | up) matrix and runs the library's one-pass SwiGLU
        # kernel between the two fused kernels (for measuring what the epilogue fusion saves).
        self.swiglu_in_epilogue = os.environ.get("MINI_NCCL_TP_SWIGLU", "epilogue") != "separate"
        self._h = None if self.swiglu_in_epilogue else torch.empty(tokens, 2 * self.ffn_local, dtype=torch.bfloat16, device="cuda")

    @property
    def input_shard(self):
        """Write this rank's tokens [M/R, H] here (it is the local part of the gather buffer)."""
        return self.ag_gemm.local_shard

    def forward(self, out=None):
        if self.swiglu_in_epilogue:
            self.ag_gemm(self.w_gate_up, out=self._act, swiglu=True)
        else:
            h = self.ag_gemm(self.w_gate_up, out=self._h)
            gate, up = split_gate_up(h)  # views; the one-pass kernel wants (gate | up) halves
            swiglu_bf16(torch.cat((gate, up), dim=1), out=self._act)
        return self.gemm_rs(self._act, self.w_down, out=out)

    def forward_unfused(self, x_shard, group=None):
        """The same block with library pieces: NCCL all-gather, cuBLAS GEMMs, NCCL reduce-scatter."""
        import torch.distributed as dist

        R = self.comm.size
        if R > 1:
            full = torch.empty(self.tokens, self.hidden, dtype=torch.bfloat16, device="cuda")
            dist.all_gather_into_tensor(full, x_shard, group=group)
        else:
            full = x_shard
        h = full @ self.w_gate_up_plain.t()
        act = F.silu(h[:, :self.ffn_local]) * h[:, self.ffn_local:]
        y = act @ self.w_down.t()
        if R == 1:
            return y
        out = torch.empty(self.tokens // R, self.hidden, dtype=torch.bfloat16, device="cuda")
        dist.reduce_scatter_tensor(out, y, group=group)
        return out


class TensorParallelAttnOut:
    """Attention output projection: heads are sharded, so the projection's K dimension is."""

    def __init__(self, comm, tokens: int, hidden: int, seed: int = 1):
        R = comm.size
        self.comm, self.tokens, self.hidden, self.k_local = comm, tokens, hidden, hidden // R
        g = torch.Generator(device="cuda").manual_seed(seed * 1000 + comm.rank)
        self.w_o = (torch.randn(hidden, self.k_local, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
        self.gemm_rs = GemmReduceScatter(comm, tokens, hidden)

    def forward(self, attn_local, out=None):
        return self.gemm_rs(attn_local, self.w_o, out=out)

    def forward_unfused(self, attn_local, group=None):
        import torch.distributed as dist

        y = attn_local @ self.w_o.t()
        if self.comm.size == 1:
            return y
        out = torch.empty(self.tokens // self.comm.size, self.hidden, dtype=torch.bfloat16, device="cuda")
        dist.reduce_scatter_tensor(out, y, group=group)
        return out
