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

from ._lib import RingPos, check, lib
from .attention import CoDAGQALandmarkPerf2
from .state import CoDAGQALandmarkStatePerf2


class CoDAStack(nn.Module):
    def __init__(self, layers: List[CoDAGQALandmarkPerf2]):
        super().__init__()
        self.layers = nn.ModuleList(layers)
        self._graph = None
        # Captured decode step: route every layer's evicted token on a second branch of the graph, beside the
        # projection GEMMs, instead of inside the layer's own chain (set before the first step_graph).
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
        g = torch.cuda.CUDAGraph()
        branch = torch.cuda.Stream(device=dev)
        with torch.cuda.graph(g):
            main = torch.cuda.current_stream(dev)
            # Routing of the tokens this step evicts needs the states only: every layer's goes to a second branch
            # of the graph at once, and each layer's new token waits for its own layer's routing.
            routed = []
            if self.split_routing:
                branch.wait_stream(main)
                with torch.cuda.stream(branch):
                    for layer, st, rp in zip(self.layers, states, rps):
                        done = None
                        if layer.route_launch(x_static.dtype, st, rp, branch.cuda_stream):
                            done = torch.cuda.Event()
                            done.record(branch)
                        routed.append(done)
            else:
                routed = [None] * len(self.layers)
            h = x_static
            for layer, st, rp, done in zip(self.layers, states, rps, routed):
                if done is not None:
                    main.wait_event(done)
                h = h + layer.step_graphable(h, st, rp, routed=done is not None)
            if self.split_routing:
                main.wait_stream(branch)
            check(lib.coda_b200_advance_steps(ctr.data_ptr(), 1, torch.cuda.current_stream(dev).cuda_stream),
                  "coda_b200_advance_steps")
            out_static = h
        self._graph = (g, x_static, out_static, ctr, [id(s) for s in states])

    @torch.no_grad()
    def step_graph(self, x: torch.Tensor, states) -> torch.Tensor:
        """Replay the captured step on ``x`` (captures on first use).  Returns the stack's static output
        buffer, which the next replay overwrites."""
        if self._graph is None or self._graph[4] != [id(s) for s in states]:
            self.capture_step(states, x)
        g, x_static, out_static, _, _ = self._graph
        x_static.copy_(x, non_blocking=True)
        g.replay()
        for layer, st in zip(self.layers, states):
            layer.advance_host_scalars(st)
        return out_static
