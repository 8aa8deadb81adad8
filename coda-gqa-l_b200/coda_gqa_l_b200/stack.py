"""A stack of bounded-cache layers driven token by token or block by block.

The harness convention (used identically by the oracle-side comparison in the tests and the benchmark)
is a residual chain ``h <- h + layer_i(h)``.  Decode steps can be captured once into a CUDA graph and
replayed: the per-step ring scalars are derived on the device from a step counter, so nothing has to be
re-captured as positions advance.  One process drives one GPU; a multi-GPU job shards the batch of
independent states across ranks and needs no collective on this path.
"""
from __future__ import annotations

import ctypes as C
import operator
from typing import List, Optional

import torch
import torch.nn as nn
from torch.nn.modules import module as _nn_module

from ._lib import RingPos, StatePtrs, check, lib
from .attention import CoDAGQALandmarkPerf2
from .state import CoDAGQALandmarkStatePerf2


# A captured step is keyed on the parameters its weight copies come from.  Reading 32 layers' parameters through
# ``nn.Module`` attribute look-ups before every replay costs more host time than the launch itself, so the stack
# keeps the Parameter objects in a flat tuple and lets ``map`` read their version counters and addresses; the
# tuple is rebuilt whenever any module of the process registers a parameter or a sub-module (an epoch that torch's
# registration hooks advance), which is what replacing a Parameter object instead of writing into it does.
_REGISTRATION_EPOCH = [0]


def _bump_epoch(*_args):
    _REGISTRATION_EPOCH[0] += 1
    return None


_nn_module.register_module_parameter_registration_hook(_bump_epoch)
_nn_module.register_module_module_registration_hook(_bump_epoch)
_version_of = operator.attrgetter("_version")
_switches_of = operator.attrgetter("use_tuned_kernels", "fuse_append_into_attention", "use_skinny_gemm_kernel",
                                   "use_skinny_in_proj", "use_own_gemm")
_banks_of = operator.attrgetter("active_exact", "active_summary")


class CoDAStack(nn.Module):
    """``residual=True`` chains the layers as ``h <- h + layer(h)``; ``residual=False`` as ``h <- layer(h)`` (a single
    layer then returns exactly what ``layer.step`` / ``layer.prefill_chunked`` return)."""

    def __init__(self, layers: List[CoDAGQALandmarkPerf2], residual: bool = True):
        super().__init__()
        self.layers = nn.ModuleList(layers)
        self.residual = bool(residual)
        self._graph = None
        self._watch = None                       # (epoch, layers, versioned tensors, addressed tensors)
        # Captured decode step: route every layer's evicted token in one launch at the start of the step instead of
        # inside each layer's own chain (set before the first step_graph).
        self.split_routing = True
        # Captured decode step: a layer's output projection and the next layer's input projection as ONE launch
        # (coda_b200_skinny_gemm_chain) wherever every layer can (set before the first step_graph).  Off: two
        # launches chained by programmatic dependent launch measure faster (1.21 against 1.32 ms per C4 step).
        self.chain_projections = False

    def init_states(self, *, batch_size: int, device, dtype) -> List[CoDAGQALandmarkStatePerf2]:
        return [l.init_state(batch_size=batch_size, device=device, dtype=dtype) for l in self.layers]

    @torch.no_grad()
    def prefill(self, x: torch.Tensor, states, *, block_size: int = 256, return_outputs: bool = True):
        """Layer by layer over the whole chunk ``x`` (B, L, D)."""
        h = x
        for i, (layer, st) in enumerate(zip(self.layers, states)):
            if self.residual:
                # the residual rides in the output projection; from the second layer on into h's own memory
                # (the first layer's h is the caller's tensor)
                h = layer.prefill_chunked_residual(h, st, block_size=block_size, inplace=i > 0)
            else:
                h, _ = layer.prefill_chunked(h, st, block_size=block_size)
        self._graph = None                       # scalars baked into a captured step are stale now
        return h if return_outputs else None

    @torch.no_grad()
    def step(self, x: torch.Tensor, states) -> torch.Tensor:
        """One decode token per state through every layer (eager launches)."""
        h = x
        for layer, st in zip(self.layers, states):
            h = layer.step_residual(h, st) if self.residual else layer.step(h, st)[0]
        self._graph = None                       # the captured step's device counter did not see this write
        return h

    # ------------------------------------------------------------------ CUDA-graph decode
    @torch.no_grad()
    def capture_step(self, states, example_x: torch.Tensor, warmup: int = 2) -> None:
        """Capture one decode step of the whole stack.  The states' contents are preserved: the warm-up
        steps run on the live buffers and are undone by restoring a snapshot of every arena."""
        dev = states[0].k_buf.device
        example_x = example_x.to(dev)
        snaps = [(st._arena.clone() if st._arena is not None else None,
                  (st.pos, st.recent_idx, st.recent_filled)) for st in states]
        if any(s[0] is None for s in snaps):
            raise RuntimeError("capture_step needs arena-backed states (create them with init_state / state_from_fields)")
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(warmup):
                h = example_x
                for layer, st in zip(self.layers, states):
                    y, _ = layer.step(h, st)
                    h = h + y if self.residual else y
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
        n_layers = len(self.layers)
        chain = (self.chain_projections and self.residual and plan is not None and n_layers > 1
                 and x_static.dim() == 3 and x_static.shape[1] == 1 and x_static.is_contiguous()
                 and all(layer.chain_ready(x_static.shape[0], x_static.dtype, st, self.layers[i + 1] if i + 1 < n_layers else None)
                         for i, (layer, st) in enumerate(zip(self.layers, states))))
        gsync = torch.zeros(2, dtype=torch.int32, device=dev) if chain else None      # the chained launches' grid barrier
        def body(h, before_layers=None):
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
            if before_layers is not None:
                before_layers()                      # (the host-fed graph joins its input copy here)
            if chain:
                # per layer: attention (writes the new token) -> [output projection + residual | next layer's input
                # projection] in one launch; the first layer's input projection is a launch of its own
                proj_y = None
                for i, (layer, st, rp) in enumerate(zip(self.layers, states, rps)):
                    h, proj_y = layer.step_chained(h, st, rp, rope_cs=rope_cs, proj_y=proj_y,
                                                   next_layer=self.layers[i + 1] if i + 1 < n_layers else None, gsync=gsync)
            else:
                for layer, st, rp in zip(self.layers, states, rps):
                    h = layer.step_graphable(h, st, rp, routed=plan is not None, residual=h if self.residual else None,
                                             rope_cs=rope_cs)
            check(lib.coda_b200_advance_steps(ctr.data_ptr(), 1, torch.cuda.current_stream(dev).cuda_stream),
                  "coda_b200_advance_steps")
            return h

        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out_static = body(x_static)
        # The same step with its host traffic inside the graph: pinned input -> device, the step, result -> pinned
        # output.  One launch per token for a caller that feeds tokens from the host (step_graph_host); both graphs
        # advance the same device counter, so replays of either may be mixed.
        x_pin = torch.empty(x_static.shape, dtype=x_static.dtype).pin_memory()
        x_pin.copy_(x_static)
        out_pin = torch.empty(out_static.shape, dtype=out_static.dtype).pin_memory()
        gh = torch.cuda.CUDAGraph()
        copy_stream = torch.cuda.Stream(device=dev)
        with torch.cuda.graph(gh):
            # the routing launch and the cos / sin table need the states only: the input's copy from the host is a
            # branch of its own beside them and joins ahead of the first layer
            cur = torch.cuda.current_stream(dev)
            copy_stream.wait_stream(cur)
            with torch.cuda.stream(copy_stream):
                x_static.copy_(x_pin, non_blocking=True)
            out_h = body(x_static, before_layers=lambda: cur.wait_stream(copy_stream))
            out_pin.copy_(out_h, non_blocking=True)
        # Everything the graph's launches point at is kept alive with it (plan, table, the layers' derived weight and
        # constant tensors), and what they were is noted so that a replay after any of them changed re-captures.
        self._graph = dict(graph=g, x=x_static, out=out_static, ctr=ctr, plan=plan, rope_cs=rope_cs, gsync=gsync, chained=chain,
                           host_graph=gh, x_pin=x_pin, out_pin=out_pin, out_host_dev=out_h,
                           states=list(states), key=self._graph_key(states, x_static.dtype),
                           expect=[(st.pos, st.recent_idx, st.recent_filled) for st in states],
                           keep=[(l._fused, l._wt, l._const_cache.get("k"), l._qrec, l._status) for l in self.layers])

    def _graph_key(self, states, dtype):
        """What a captured step depends on besides the ring scalars, cheap enough to evaluate before every replay:
        the state objects and their active bank sizes, the layers' switches, and address + version counter of the
        parameters the derived weight copies and constants are built from (``load_state_dict``, in-place updates and
        ``.to()`` all move one of the two).  After writing a parameter through ``.data`` call :meth:`invalidate`."""
        w = self._watch
        if w is None or w[0] != _REGISTRATION_EPOCH[0]:
            layers = tuple(self.layers)
            weights = tuple(t for l in layers for t in (l.q_proj.weight, l.o_proj.weight))
            w = self._watch = (_REGISTRATION_EPOCH[0], layers,
                               weights + tuple(t for l in layers for t in (l.theta, l.summary_eta_logit)), weights)
        return (self.split_routing, self.chain_projections, self.residual, dtype, w[0], tuple(map(_version_of, w[2])),
                tuple(map(torch.Tensor.data_ptr, w[3])), tuple(map(_switches_of, w[1])),
                tuple(map(id, states)), tuple(map(_banks_of, states)))

    def invalidate(self) -> None:
        """Drop the captured step (the next :meth:`step_graph` captures again)."""
        self._graph = None

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
    def _live_graph(self, x: torch.Tensor, states):
        """The captured step for these states, re-captured when it no longer describes them."""
        G = self._graph
        if G is not None:
            # Ring scalars are baked at capture time and advanced by the graph's own device counter, so a write that
            # did not go through a replay (an eager step or prefill on one of the layers, a restored state) makes
            # the graph stale; so does any rebuilt weight copy or constant.  Either way: capture again.
            if (len(G["states"]) != len(states) or any(map(operator.is_not, G["states"], states))
                    or G["expect"] != [(st.pos, st.recent_idx, st.recent_filled) for st in states]
                    or G["key"] != self._graph_key(states, x.dtype)
                    or x.shape != G["x"].shape or x.dtype != G["x"].dtype):
                G = None
        if G is None:
            self.capture_step(states, x)
            G = self._graph
        return G

    def _replayed(self, G, states) -> None:
        for layer, st in zip(self.layers, states):
            layer.advance_host_scalars(st)
        G["expect"] = [(st.pos, st.recent_idx, st.recent_filled) for st in states]

    def step_graph(self, x: torch.Tensor, states) -> torch.Tensor:
        """Replay the captured step on ``x`` (captures on first use).  Returns the stack's static output
        buffer, which the next replay overwrites."""
        G = self._live_graph(x, states)
        G["x"].copy_(x, non_blocking=True)
        G["graph"].replay()
        self._replayed(G, states)
        return G["out"]

    def step_graph_host(self, x_host: torch.Tensor, states) -> torch.Tensor:
        """One decode step fed from and answered to the host in ONE launch: ``x_host`` (a CPU tensor) is copied into
        the stack's pinned input buffer, and the replayed graph carries the host-to-device copy, the step and the
        device-to-host copy of the result.  Returns the pinned CPU output buffer; it is valid once the current stream
        has been synchronised and is overwritten by the next call (so synchronise before calling again: the input
        buffer is rewritten by the host at once)."""
        G = self._live_graph(x_host, states)
        G["x_pin"].copy_(x_host)
        G["host_graph"].replay()
        self._replayed(G, states)
        return G["out_pin"]
