"""Host-buffer front end: run a per-case callable on tensors that live in pinned host memory.

The reference's callables take device tensors (cases/kernels/h2o.py:41-58 creates its inputs on the
GPU); a host application that keeps its activations in host memory pays a host->device copy of
q, k, v and a device->host copy of every output around each call.  At the benchmark shapes those
copies take several times longer than the kernels, so running them back to back on one stream
leaves both the copy engines and the SMs idle most of the time.  ``HostPipeline`` keeps ``depth``
calls in flight: inputs are staged on a copy-in stream, the case runs on a compute stream, results
leave on a copy-out stream, and CUDA events order the three per slot.  With depth >= 2 a steady
stream of calls is bound by the slower copy direction alone.

Only plumbing lives here (streams, events, staging buffers); the arithmetic is the case's own.
"""
from typing import Callable, List, Sequence

import torch


class HostPipeline:
  """``submit(host_inputs, host_outputs)`` enqueues one call; ``drain()`` waits for all of them.

  ``fn`` is a per-case callable taking device tensors positionally and returning a tensor or a
  tuple of tensors.  ``host_inputs`` / ``host_outputs`` are sequences of pinned CPU tensors; the
  outputs must match the shapes and dtypes ``fn`` returns.  The caller must not touch a call's host
  buffers until ``drain()`` (or ``wait(ticket)``) has returned.
  """

  def __init__(self, fn: Callable, example_inputs: Sequence[torch.Tensor], depth: int = 2, device=None):
    if depth < 1:
      raise ValueError("depth must be >= 1")
    self.fn = fn
    self.depth = depth
    self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(self.device):
      self.s_in = torch.cuda.Stream()
      self.s_run = torch.cuda.Stream()
      self.s_out = torch.cuda.Stream()
      self.dev_in: List[List[torch.Tensor]] = [
          [torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in example_inputs] for _ in range(depth)]
      mk = lambda: [torch.cuda.Event() for _ in range(depth)]
      self.in_done, self.run_done, self.out_done = mk(), mk(), mk()
    self.live = [None] * depth   # device outputs of the call that last used the slot
    self.used = [False] * depth
    self.n = 0

  def begin(self):
    """Order everything submitted from now on after the work already on the current stream."""
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream(self.device))
    for s in (self.s_in, self.s_run, self.s_out):
      s.wait_event(ev)

  def submit(self, host_inputs: Sequence[torch.Tensor], host_outputs: Sequence[torch.Tensor]) -> int:
    for t in list(host_inputs) + list(host_outputs):
      if t.is_cuda or not t.is_pinned():
        raise ValueError("HostPipeline takes pinned host tensors")
    slot = self.n % self.depth
    if self.used[slot]:
      # the slot's previous results must have left the device before their tensors are released
      self.out_done[slot].synchronize()
      self.live[slot] = None
    with torch.cuda.device(self.device):
      with torch.cuda.stream(self.s_in):
        if self.used[slot]:
          self.s_in.wait_event(self.run_done[slot])   # the previous call read these staging buffers
        for d, h in zip(self.dev_in[slot], host_inputs):
          d.copy_(h, non_blocking=True)
        self.in_done[slot].record(self.s_in)
      with torch.cuda.stream(self.s_run):
        self.s_run.wait_event(self.in_done[slot])
        outs = self.fn(*self.dev_in[slot])
        outs = (outs,) if torch.is_tensor(outs) else tuple(outs)
        self.run_done[slot].record(self.s_run)
      if len(outs) != len(host_outputs):
        raise ValueError(f"the case returns {len(outs)} tensors, {len(host_outputs)} host buffers given")
      with torch.cuda.stream(self.s_out):
        self.s_out.wait_event(self.run_done[slot])
        for h, o in zip(host_outputs, outs):
          h.copy_(o, non_blocking=True)
        self.out_done[slot].record(self.s_out)
    self.live[slot] = outs
    self.used[slot] = True
    self.n += 1
    return self.n - 1

  def join(self):
    """Make the current stream wait for every call submitted so far (no host synchronisation)."""
    cur = torch.cuda.current_stream(self.device)
    for slot in range(self.depth):
      if self.used[slot]:
        cur.wait_event(self.out_done[slot])

  def drain(self):
    """Block the host until every submitted call has delivered its outputs."""
    for slot in range(self.depth):
      if self.used[slot]:
        self.out_done[slot].synchronize()
        self.live[slot] = None


class GraphedCall:
  """``GraphedCall(fn)(*inputs)``: the kernels of ``fn(*inputs)`` recorded once per distinct set of
  input tensors into a CUDA graph, replayed on every later call with the same tensors.

  A call of a case through the operator layer costs the host 20-70 microseconds (descriptors,
  output allocation, one to four launches); at small shapes, or with a configuration's (batch,
  head) units spread over several GPUs, that is more than the kernels take.  A replay costs the
  host one launch.  The graph reads the very tensors it was recorded with -- the caller refreshes
  their contents in place -- and every replay overwrites the outputs of the one before: what a
  call returns is valid until the next call with the same inputs.  Inputs are told apart by
  address, shape, strides and dtype; at most ``max_graphs`` graphs are kept, the least recently
  used one is dropped.

  Replays run on the stream that is current at the call.  ``launches`` counts the kernels
  replayed so far (as recorded by the library's own launch counter while capturing).
  """

  def __init__(self, fn: Callable, max_graphs: int = 8, warmup: int = 2):
    self.fn, self.max_graphs, self.warmup = fn, max_graphs, warmup
    self.cache = {}      # key -> (graph, outputs, launches, inputs kept alive)
    self.launches = 0

  @staticmethod
  def _key(inputs):
    return tuple((t.data_ptr(), tuple(t.shape), t.stride(), t.dtype) for t in inputs)

  def _record(self, inputs):
    from . import ops
    dev = inputs[0].device
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
      for _ in range(self.warmup):     # first-call set-up (function attributes, workspaces) happens here
        self.fn(*inputs)
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    before = ops.launch_count()
    with torch.cuda.graph(graph, stream=side):
      outs = self.fn(*inputs)
    launches = ops.launch_count() - before
    torch.cuda.current_stream(dev).wait_stream(side)
    return graph, outs, launches, tuple(inputs)

  def __call__(self, *inputs):
    key = self._key(inputs)
    entry = self.cache.pop(key, None)
    if entry is None:
      if len(self.cache) >= self.max_graphs:
        self.cache.pop(next(iter(self.cache)))
      entry = self._record(inputs)
    self.cache[key] = entry              # (re-inserted last: most recently used)
    entry[0].replay()
    self.launches += entry[2]
    return entry[1]
