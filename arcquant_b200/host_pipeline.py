"""Quantizing activations that live in host memory.

The reference's operators take device tensors; a caller whose activations sit in (pinned) host
memory pays a host->device copy of 2*KQ bytes per token before the kernel and a device->host copy of
the packed result after it, and on a PCIe-attached GPU those copies, not the kernel, set the pace.
`HostQuantizePipeline` cuts the token range into chunks that own whole 128-row scale tiles and runs
the upload of chunk i+1, the kernel of chunk i and the download of chunk i-1 on three streams, so the
two copy directions overlap each other and the kernel.  Results are byte-identical to one call on the
whole range: rows are quantized independently and a chunk's scale tiles are a contiguous slice of
the scale buffer.
"""
from __future__ import annotations

import torch

from . import ops


class HostQuantizePipeline:
    def __init__(self, tokens: int, kq: int, ke: int, device, chunk_rows: int = 4096, buffers: int = 3):
        if chunk_rows % 128:
            raise ValueError("chunk_rows must be a multiple of 128 (whole scale tiles)")
        self.tokens, self.kq, self.ke = tokens, kq, ke
        self.k_eff = kq + ke
        self.dev = torch.device(device)
        self.chunk = min(chunk_rows, ((tokens + 127) // 128) * 128)
        self.nbuf = buffers
        self.tile_bytes = ((self.k_eff // 16 + 3) // 4) * 512          # scale bytes of one 128-row tile
        with torch.cuda.device(self.dev):
            self.dx = [torch.empty((self.chunk, kq), dtype=torch.bfloat16, device=self.dev) for _ in range(buffers)]
            self.dq = [torch.empty((self.chunk, self.k_eff // 2), dtype=torch.uint8, device=self.dev)
                       for _ in range(buffers)]
            self.dsf = [torch.empty((ops.sf_bytes(self.chunk, self.k_eff),), dtype=torch.uint8, device=self.dev)
                        for _ in range(buffers)]
            self.s_in, self.s_k, self.s_out = (torch.cuda.Stream(self.dev) for _ in range(3))
            self.ev_in = [torch.cuda.Event() for _ in range(buffers)]
            self.ev_k = [torch.cuda.Event() for _ in range(buffers)]
            self.ev_out = [torch.cuda.Event() for _ in range(buffers)]

    def sf_bytes(self) -> int:
        return ops.sf_bytes(self.tokens, self.k_eff)

    @torch.no_grad()
    def run(self, hx: torch.Tensor, reorder_index, hq: torch.Tensor, hsf: torch.Tensor, gamma=None, eps: float = 0.0):
        """hx [tokens, KQ] bf16, hq [tokens, K_eff/2] u8, hsf [sf_bytes()] u8: pinned host tensors.
        gamma given -> fused RMSNorm.  Returns after everything has landed in hq / hsf."""
        cur = torch.cuda.current_stream(self.dev)
        for s in (self.s_in, self.s_k, self.s_out):
            s.wait_stream(cur)
        nchunks = (self.tokens + self.chunk - 1) // self.chunk
        for c in range(nchunks):
            b = c % self.nbuf
            r0 = c * self.chunk
            rows = min(self.chunk, self.tokens - r0)
            with torch.cuda.stream(self.s_in):
                if c >= self.nbuf:
                    self.s_in.wait_event(self.ev_k[b])        # the kernel that read dx[b] is done
                self.dx[b][:rows].copy_(hx[r0:r0 + rows], non_blocking=True)
                self.ev_in[b].record(self.s_in)
            with torch.cuda.stream(self.s_k):
                self.s_k.wait_event(self.ev_in[b])
                if c >= self.nbuf:
                    self.s_k.wait_event(self.ev_out[b])       # the download of dq[b] / dsf[b] is done
                out = (self.dq[b], self.dsf[b])
                if gamma is None:
                    ops.reorder_quantize_x(self.dx[b][:rows], reorder_index, self.ke, out=out)
                else:
                    ops.rmsnorm_quantize_x(self.dx[b][:rows], gamma, eps, reorder_index, self.ke, out=out)
                self.ev_k[b].record(self.s_k)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_k[b])
                hq[r0:r0 + rows].copy_(self.dq[b][:rows], non_blocking=True)
                nsf = ((rows + 127) // 128) * self.tile_bytes
                o = (r0 // 128) * self.tile_bytes
                hsf[o:o + nsf].copy_(self.dsf[b][:nsf], non_blocking=True)
                self.ev_out[b].record(self.s_out)
        for s in (self.s_in, self.s_k, self.s_out):
            cur.wait_stream(s)
        cur.synchronize()
