"""Tensor-parallel (Megatron-style, sequence-parallel) MLP and attention-output blocks built on the
fused kernels.  Activations between blocks are sharded by tokens (M / ranks rows per rank); weights
are sharded along the hidden FFN dimension.

  MLP:   X_r [M/R, H]  --all-gather->GEMM-->  [M, 2F/R] (gate | up)  --SwiGLU-->  [M, F/R]
                       --GEMM->reduce-scatter-->  Y_r [M/R, H]
  attention output projection:  A [M, H/R]  --GEMM->reduce-scatter-->  Y_r [M/R, H]

The reference has no model or parallelism code; the shapes are those of the tensor-parallel
benchmark configuration (Llama-3-8B: H = 4096, F = 14336, TP = 8, 4096 tokens)."""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F

from ..ops.elementwise import swiglu_bf16
from ..ops.fused import AllGatherGemm, GemmReduceScatter


class TensorParallelMLP:
    def __init__(self, comm, tokens: int, hidden: int, ffn: int, seed: int = 0, n_comm_ctas: int = 0):
        R = comm.size
        if ffn % R:
            raise ValueError("ffn must divide by the number of ranks")
        self.comm, self.tokens, self.hidden, self.ffn_local = comm, tokens, hidden, ffn // R
        g = torch.Generator(device="cuda").manual_seed(seed * 1000 + comm.rank)
        std = 0.02
        # nn.Linear layout [out_features, in_features]; gate and up stacked along out_features
        self.w_gate_up = (torch.randn(2 * self.ffn_local, hidden, generator=g, device="cuda") * std).to(torch.bfloat16)
        self.w_down = (torch.randn(hidden, self.ffn_local, generator=g, device="cuda") * std).to(torch.bfloat16)
        self.ag_gemm = AllGatherGemm(comm, tokens, hidden, n_comm_ctas=n_comm_ctas)
        self.gemm_rs = GemmReduceScatter(comm, tokens, hidden)
        self._h = torch.empty(tokens, 2 * self.ffn_local, dtype=torch.bfloat16, device="cuda")
        self._act = torch.empty(tokens, self.ffn_local, dtype=torch.bfloat16, device="cuda")
        # SwiGLU between the two fused kernels: the library's one-pass kernel (MINI_NCCL_TP_FUSED_SWIGLU=1)
        # or the framework's silu and mul (default)
        self.fused_swiglu = os.environ.get("MINI_NCCL_TP_FUSED_SWIGLU", "0") == "1" and self.ffn_local % 8 == 0

    @property
    def input_shard(self):
        """Write this rank's tokens [M/R, H] here (it is the local part of the gather buffer)."""
        return self.ag_gemm.local_shard

    def forward(self, out=None):
        h = self.ag_gemm(self.w_gate_up, out=self._h)
        if self.fused_swiglu:
            swiglu_bf16(h, out=self._act)  # one pass, one rounding
        else:
            gate, up = h[:, :self.ffn_local], h[:, self.ffn_local:]
            torch.mul(F.silu(gate), up, out=self._act)
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
        h = full @ self.w_gate_up.t()
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
