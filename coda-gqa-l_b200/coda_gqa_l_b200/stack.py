"""A stack of bounded-cache layers driven token by token or block by block.

The harness convention (used identically by the oracle-side comparison in the tests and the benchmark)
is a residual chain ``h <- h + layer_i(h)``.  Decode steps can be captured once into a CUDA graph and
replayed: the per-step ring scalars are derived on the device from a step counter, so nothing has to be
re-captured as positions advance.  One process drives one GPU; a multi-GPU job shards the batch of
independent states across ranks and needs no collective on this path.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch
import torch.nn as nn

from ._lib import RingPos, StatePtrs, check, lib
from .attention import CoDAGQALandmarkPerf2
from .state import CoDAGQALandmarkStatePerf2


class CoDAStack(nn.Module):
    def __init__(self, layers: List[CoDAGQALandmarkPerf2]):
        super().__init__()
        self.layers = nn.ModuleList(layers)
        self._graph = None
        # Captured decode step: route every layer's evicted token in one launch at the start of the step instead of
        # inside each layer's own chain (set before the first step_graph).
        self.split_routing = True

    def init_states(self, *, batch_size: int, device, dtype) -> List[CoDAGQALandmarkStatePerf2]:
        return [l.init_state(batch_size=batch_size, device=device, dtype=dtype) for l in self.layers]

    @torch.no_grad()
    def prefill(self, x: torch.Tensor, states, *, block_size: int = 256, return_outputs: bool = True):
        """Layer by layer over the whole chunk ``x`` (B, L, D)."""
        h = x
        for layer, st in zip(self.layers, states):
            y, _ = layer.prefill_chunked(h, st, block_size=block_size)
            h = h + y
        self._graph = None                       # scalars baked into a captured step are stale now
        return h if return_outputs else None

    @torch.no_grad()
    def step(self, x: torch.Tensor, states) -> torch.Tensor:
        """One decode token per state through every layer (eager launches)."""
        h = x
        for layer, st in zip(self.layers, states):
            y, _ = layer.step(h, st)
            h = h + y
        return h

    # ------------------------------------------------------------------ CUDA-graph decode
    @torch.no_grad()
    def capture_step(self, states, example_x: torch.Tensor, warmup: int = 2) -> None:
        """Capture one decode step of the whole stack.  The states' contents are preserved: the warm-up
        steps run on the live buffers and are undone by restoring a snapshot of every arena."""
        dev = example_x.device
        snaps = [(st._arena.clone() if st._arena is not None else None,
                  (st.pos, st.recent_idx, st.recent_filled)) for st in states]
        if any(s[0] is None for s in snaps):
            raise RuntimeError("capture_step needs arena-backed states (create them with init_state / state_from_fields)")
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self.step(example_x, states)
        torch.cuda.current_stream(dev).wait_stream(side)
        for st, (arena, sc) in zip(states, snaps):
            st._arena.copy_(arena)
            st.pos, st.recent_idx, st.recent_filled = sc
        ctr = torch.zeros(1, dtype=torch.int64, device=dev)
        x_static = example_x.clone()
        rps = [RingPos(int(st.pos), int(st.recent_idx), int(st.recent_filled), ctr.data_ptr()) for st in states]
        plan = self._route_plan(states, rps, x_static.dtype) if self.split_routing else None
        rope_cs = None
        if plan is not None and self._shared_rope(states, x_static.dtype):      # (compares tensors: outside the capture)
            rope_cs = torch.empty(self.layers[0].head_dim, dtype=torch.float32, device=dev)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            # Routing of the tokens this step evicts needs the states only: all layers' in one launch up front
            # (one layer's routing is a chain of memory round trips; side by side they are bandwidth-bound), so
            # that a layer's own chain is projection -> new token's write -> attention -> output projection.
            if plan is not None:
                check(lib.coda_b200_step_route_batched(C.byref(plan[0]), plan[1].data_ptr(), len(self.layers),
                                                       torch.cuda.current_stream(dev).cuda_stream),
                      "coda_b200_step_route_batched")
            # cos / sin of this step's position: once for all layers instead of once per CTA of every layer
            if rope_cs is not None:
                l0 = self.layers[0]
                check(lib.coda_b200_rope_table(C.byref(plan[0]), rps[0], l0._consts(dev, x_static.dtype)[0].data_ptr(),
                                               rope_cs.data_ptr(), torch.cuda.current_stream(dev).cuda_stream),
                      "coda_b200_rope_table")
            h = x_static
            for layer, st, rp in zip(self.layers, states, rps):
                h = layer.step_graphable(h, st, rp, routed=plan is not None, residual=h, rope_cs=rope_cs)
            check(lib.coda_b200_advance_steps(ctr.data_ptr(), 1, torch.cuda.current_stream(dev).cuda_stream),
                  "coda_b200_advance_steps")
            out_static = h
        self._graph = (g, x_static, out_static, ctr, [id(s) for s in states], plan, rope_cs)   # plan / table live as long as the graph

    def _shared_rope(self, states, dtype) -> bool:
        """Do all layers rotate by the same angles at the same position (same head_dim, frequencies, angle dtype
        and position)?  Then one cos / sin table per step serves them all."""
        l0, s0 = self.layers[0], states[0]
        f0 = l0._consts(s0.k_buf.device, dtype)[0]
        for layer, st in zip(self.layers, states):
            f = layer._consts(st.k_buf.device, dtype)[0]
            if (layer.head_dim != l0.head_dim or st.pos != s0.pos or layer.rope.inv_freq.dtype != l0.rope.inv_freq.dtype
                    or f.shape != f0.shape or not torch.equal(f, f0)):
                return False
        return True

    def _route_plan(self, states, rps, dtype):
        """Device plan for the batched routing launch, or None where the layers do not share one configuration
        the fused cache-write kernel covers (then every layer routes inside its own step)."""
        l0 = self.layers[0]
        cfg = l0._cfg(states[0].k_buf.shape[0], dtype, states[0])
        keys = ("B", "H", "Hkv", "Dh", "W", "Me", "Ms", "dtype", "rope_interleaved", "gated", "refresh_on_hit",
                "overwrite_on_insert", "active_exact", "active_summary", "tau_gate_exact", "tau_gate_summary",
                "tau_match", "tau_novel", "energy_scale")
        for layer, st in zip(self.layers, states):
            c = layer._cfg(st.k_buf.shape[0], dtype, st)
            if any(getattr(c, k) != getattr(cfg, k) for k in keys) or layer._tracked(st):
                return None
            if not (layer._tuned_decode(c) and layer._fused_write_ok(c)):
                return None
        n = len(self.layers)
        dev = states[0].k_buf.device
        sts = (StatePtrs * n)(*[layer._ptrs(st) for layer, st in zip(self.layers, states)])
        rpa = (RingPos * n)(*rps)
        etas = (C.c_void_p * n)(*[layer._consts(dev, dtype)[3].data_ptr() for layer in self.layers])
        buf = torch.zeros(int(lib.coda_b200_step_route_plan_bytes(n)), dtype=torch.uint8, device=dev)
        check(lib.coda_b200_step_route_plan(C.byref(cfg), sts, rpa, etas, n, buf.data_ptr(),
                                            torch.cuda.current_stream(dev).cuda_stream), "coda_b200_step_route_plan")
        return cfg, buf

    @torch.no_grad()
    def step_graph(self, x: torch.Tensor, states) -> torch.Tensor:
        """Replay the captured step on ``x`` (captures on first use).  Returns the stack's static output
        buffer, which the next replay overwrites."""
        if self._graph is None or self._graph[4] != [id(s) for s in states]:
            self.capture_step(states, x)
        g, x_static, out_static = self._graph[:3]
        x_static.copy_(x, non_blocking=True)
        g.replay()
        for layer, st in zip(self.layers, states):
            layer.advance_host_scalars(st)
        return out_static
