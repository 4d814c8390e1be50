"""Recurrent (T = 1) use of the decay rule without per-step allocations.

The reference's recurrent protocol is `LFWFunction.apply` with the returned state fed back in
(t2fw/functional_lfw.py:65; its benchmark times exactly that step, tests/benchmark.py:104-105).
That call allocates its outputs, so the state changes address every step.  The additions here keep
the addresses fixed:

  lfw_decode_step(...)   one step into caller-owned `outputs` and `state_out`
  LFWDecodeLoop          two alternating state buffers, a ring of input slots, and a CUDA graph
                         over one trip round the ring, so that a decode loop costs one graph
                         launch per `ring` steps

A state produced by a T > 1 call (prefill) is handed over by passing it to the constructor.
"""
import torch

from . import _lib

_lib.load_ops()


def lfw_decode_step(x, f, query, key, f_key, state_in, state_out, outputs):
    """o = S' q with S' = (f f_key^T) * S + x key^T; writes `outputs` [B,1,D] and `state_out` [B,D,K].
    `state_out` must be a different buffer from `state_in`."""
    torch.ops.lfw.decode_step(x, f, query, key, f_key, state_in, state_out, outputs)
    return outputs, state_out


class LFWDecodeLoop:
    """Graph-replayed decode loop.

    `ring` (even) input slots x, f [ring,B,1,D] and query, key, f_key [ring,B,1,K] are filled by the
    caller; `run_ring()` advances the state by `ring` steps (slot 0 first) and leaves the outputs of
    every step in `outputs` [ring,B,1,D].  The first call runs eagerly and captures the graph; later
    calls replay it.  `state` is the current state (a view of one of the two internal buffers)."""

    def __init__(self, state, ring=2):
        if ring < 2 or ring % 2:
            raise ValueError("ring must be even and >= 2 (the state returns to its first buffer)")
        if not (state.is_cuda and state.dim() == 3):
            raise RuntimeError("state must be a CUDA tensor [B, D, K]")
        state = state.contiguous()      # `next_state` of a T > 1 call is a strided view of its checkpoints
        B, D, K = state.shape
        opt = dict(dtype=state.dtype, device=state.device)
        self.ring = ring
        self._s = [state.clone(), torch.empty_like(state)]
        self.x = torch.zeros(ring, B, 1, D, **opt)
        self.f = torch.ones(ring, B, 1, D, **opt)
        self.query = torch.zeros(ring, B, 1, K, **opt)
        self.key = torch.zeros(ring, B, 1, K, **opt)
        self.f_key = torch.ones(ring, B, 1, K, **opt)
        self.outputs = torch.empty(ring, B, 1, D, **opt)
        self._graph = None
        self.steps = 0

    @property
    def state(self):
        return self._s[0]          # after a whole trip round the ring the state is back in buffer 0

    def _trip(self):
        for i in range(self.ring):
            lfw_decode_step(self.x[i], self.f[i], self.query[i], self.key[i], self.f_key[i],
                            self._s[i & 1], self._s[(i + 1) & 1], self.outputs[i])

    def run_ring(self):
        if self._graph is None:
            self._trip()                                   # eager: also the warm-up before capture
            side = torch.cuda.Stream(self.x.device)
            side.wait_stream(torch.cuda.current_stream(self.x.device))
            g = torch.cuda.CUDAGraph()
            # capture on a side stream with throw-away state buffers: capturing does not execute,
            # but the graph must name the real buffers, so capture with them and restore nothing
            with torch.cuda.stream(side):
                with torch.cuda.graph(g, stream=side):
                    self._trip()
            torch.cuda.current_stream(self.x.device).wait_stream(side)
            self._graph = g
        else:
            self._graph.replay()
        self.steps += self.ring
        return self.outputs
