"""Captured decode steps: every launch of a step of a stack of layers in one CUDA graph.

The reference issues plan -> attention -> update as separate launches per layer and step and lists
a captured step as an open item (format37/kvskip README.md:358, docs/03-gate-digest.md:361-362): the
sequence length is a by-value launch parameter there, so a capture would be stale one token later.
Here the kernels can read the length from device memory (`t_dev`), so one capture stays valid
while the cache grows, as long as

  * k and v are views of the whole provisioned cache (their length is only a bound: it sizes the
    grids, the tensor maps and the statistics rows), and the planner state has capacity for it;
  * q, the token ids and every other per-step input live in buffers whose addresses do not change
    (the caller copies the step's values into them before `step()`);
  * the scalars of the policy that the host decides per step (the maximum age during the warm-up
    period, whether the correction is applied yet) are unchanged: `StepGraph` asks the layers
    for them before every step and captures again when they differ.

    t_dev = torch.tensor([T0], dtype=torch.int32, device="cuda")
    def launch():                      # one decode step of all layers, on the current stream
        K.ext().advance(t_dev, 1)
        K.ext().index_blocks(ids, cap, idx, t_dev)
        for layer, (k, v) in zip(layers, caches):
            outs.append(layer.step(q_buf[l], k, v, scale, idx, t_dev=t_dev))
    g = StepGraph(launch, layers)
    for _ in range(steps):
        q_buf.copy_(next_q)
        g.step()

Programmatic dependent launches are captured as such, so the overlap of a kernel's set-up with
its predecessor's tail is kept inside the graph.
"""

import torch


class StepGraph:
    """Runs `launch()` eagerly the first `eager` times (kernel attributes and the allocator warm
    up), then captures it once and replays the capture on every later `step()`.

    layers: objects with `graph_scalars()` (the host-decided scalars their next step would pass
    to the kernels) and `note_replayed()` (called once per replayed step so that their host-side
    step counters keep up); `RefreshLayer` has both.  The return value of the captured `launch()`
    (tensors in the graph's memory pool, rewritten by every replay) is returned by `step()`."""

    def __init__(self, launch, layers=(), eager: int = 1):
        self.launch = launch
        self.layers = list(layers)
        self.eager = eager
        self.graph = None
        self.result = None
        self.signature = None
        self.captures = 0
        self.replays = 0

    def _scalars(self):
        return tuple(layer.graph_scalars() for layer in self.layers)

    def invalidate(self):
        """Drop the capture (e.g. after the cache or the planner state was re-allocated)."""
        self.graph = None
        self.result = None

    def will_capture(self) -> bool:
        """True if the next `step()` records a new capture before replaying it."""
        return self.eager <= 0 and (self.graph is None or self._scalars() != self.signature)

    def step(self):
        if self.eager > 0:
            self.eager -= 1
            return self.launch()
        sig = self._scalars()
        if self.graph is None or sig != self.signature:
            for layer in self.layers:            # an `update` still in flight on a layer's own stream
                if hasattr(layer, "join"):       # is joined here: a capture cannot wait for it
                    layer.join()
            graph = torch.cuda.CUDAGraph()
            # thread-local capture mode: CUDA calls of other threads (e.g. a communication
            # library's watchdog) do not invalidate the capture
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                result = self.launch()          # recorded, not run; advances the layers' counters
            self.graph, self.result, self.signature = graph, result, sig
            self.captures += 1
        else:
            for layer in self.layers:
                layer.note_replayed()
        self.graph.replay()
        self.replays += 1
        return self.result
