"""A stack of encoder layers run through the raw (non-autograd) passes, with
data-parallel gradient reduction overlapped with the rest of backward.

The reference times one layer (pytorch_module/run_encoder.py:345-383); a BERT-large
encoder is 24 of them with independent weights.  Forward keeps every layer's
intermediates alive (one arena per layer, allocated once and reused every step);
backward walks the layers in reverse with ONE shared arena for backward
intermediates, writes layer l's 12 parameter gradients into bucket l and starts
its sum-allreduce at once, so the reduction of layer l runs beside the backward of
layer l-1 (parameter gradients become final in the order
DS2,DB2 -> DLINW2 -> ... -> DWKQV -> DBKQV, i.e. at the end of the layer's backward).
"""

import torch

from . import layouts as L
from .data_parallel import GradientBucketReducer
from .encoder import Encoder


class EncoderStack:
    def __init__(self, num_layers, batch_size, max_seq_len, num_heads, embedding_size, layouts,
                 dropout_p=0.1, device='cuda', mask_mode='philox', seed=0, activation='relu',
                 weight_std=0.02, group=None, dtype=torch.float16):
        self.device = torch.device(device)
        self.layers = []
        gen = torch.Generator(device=self.device).manual_seed(seed)
        for l in range(num_layers):
            enc = Encoder('', batch_size, max_seq_len, num_heads, embedding_size, layouts, dtype,
                          dropout_p, dropout_p, dropout_p, dropout_p, mask_mode=mask_mode, seed=seed + l,
                          activation=activation).to(self.device)
            with torch.no_grad():
                for (name, _), prm in zip(layouts['params'], enc.params):
                    if name in ('WKQV', 'WO', 'LINW1', 'LINW2'):
                        prm.copy_((torch.randn(prm.shape, device=self.device, generator=gen) * weight_std).to(dtype))
                    elif name in ('S1', 'S2'):
                        prm.fill_(1.0)
                    else:
                        prm.zero_()
            self.layers.append(enc)
        e0 = self.layers[0]
        self.table = L.validate(layouts)
        shape_x = L.shape_of(self.table['X'], e0.sizes)
        self.weights = [[p.detach() for p in enc.params] for enc in self.layers]
        self.fwd = [enc.views('forward', torch.empty(enc.arena_bytes('forward'), dtype=torch.uint8, device=self.device))
                    for enc in self.layers]
        self.bwd = e0.views('backward', torch.empty(e0.arena_bytes('backward'), dtype=torch.uint8, device=self.device))
        # activations between layers: acts[l] is the input of layer l, acts[-1] the output
        self.acts = [torch.empty(shape_x, dtype=dtype, device=self.device) for _ in range(num_layers + 1)]
        self.dacts = [torch.empty(shape_x, dtype=dtype, device=self.device) for _ in range(2)]
        self.reducer = GradientBucketReducer(e0.arena_bytes('grads'), self.device, group=group, buffers=num_layers, dtype=dtype)
        self.grads = [enc.views('grads', self.reducer.arenas[l]) for l, enc in enumerate(self.layers)]
        if mask_mode == 'explicit':
            raise NotImplementedError('the stack draws its masks in the kernels (Philox); explicit masks are a '
                                      'single-layer testing facility')

    def memory_bytes(self):
        e0 = self.layers[0]
        return (len(self.layers) * (e0.arena_bytes('forward') + e0.arena_bytes('grads')) + e0.arena_bytes('backward'))

    def forward(self, X):
        self.acts[0].copy_(X)
        for l, enc in enumerate(self.layers):
            enc.forward_raw(self.acts[l], self.weights[l], self.fwd[l], self.acts[l + 1])
        return self.acts[-1]

    def backward(self, DY, trace=None):
        """Returns dX; gradients of layer l are in ``self.grads[l]`` once ``wait_gradients`` returns.

        ``trace``: an empty list to be filled with one (layer, event at the end of that layer's backward, event at
        the end of its bucket's allreduce or None) per layer, plus a leading ('start', event, None): what
        ``overlap_trace`` turns into times.  The allreduce events are recorded on a stream of their own that
        waits for each reduction in turn, so tracing does not change what the compute stream waits for."""
        cur = DY
        tracing = trace is not None and self.device.type == 'cuda'
        if tracing:
            if self.__dict__.get('_trace_stream') is None:
                self._trace_stream = torch.cuda.Stream(self.device)
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            trace.append(('start', ev, None))
        for l in range(len(self.layers) - 1, -1, -1):
            self.reducer.wait(l)                         # bucket l free again (previous step's reduction done)
            out = self.dacts[l & 1]
            self.layers[l].backward_raw(cur, self.grads[l], self.bwd, self.weights[l], self.fwd[l], self.acts[l], out)
            if tracing:
                done = torch.cuda.Event(enable_timing=True)
                done.record()
            self.reducer.reduce_async(l)
            if tracing:
                reduced = None
                works = self.reducer.pending[l % len(self.reducer.arenas)]
                if works:
                    with torch.cuda.stream(self._trace_stream):
                        for w in works:
                            w.wait()
                        reduced = torch.cuda.Event(enable_timing=True)
                        reduced.record()
                trace.append((l, done, reduced))
            cur = out
        return cur

    @staticmethod
    def overlap_trace(trace):
        """Times in ms since the start of the traced backward: [[layer, backward done, allreduce done or None], ...]
        in the order the layers ran (last layer first).  Call after the device has finished the step."""
        start = trace[0][1]
        return [[l, round(start.elapsed_time(done), 3), None if red is None else round(start.elapsed_time(red), 3)]
                for l, done, red in trace[1:]]

    def wait_gradients(self):
        self.reducer.drain()
