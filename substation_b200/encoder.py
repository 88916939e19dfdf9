"""PyTorch interface to the B200 encoder layer: a drop-in for the reference's
``pytorch_module/encoder.py``.

Same class name, positional signature, parameter names/shapes, ``.params``,
``.layouts``, ``.debug`` and autograd behaviour (``backward`` returns
``(DX, *parameter gradients)`` in the configuration's order); underneath, one
ctypes call per pass into the hand-written sm_100a library instead of a
per-configuration nvcc build (pytorch_module/encoder.py:165-405).

What differs, on purpose:
  * ``torch.float16`` and ``torch.bfloat16`` are implemented (16-bit storage, fp32 accumulation; one build of
    the library per storage type), ``float32`` / ``float64`` are not;
  * dropout masks are ``uint8``; with ``mask_mode='explicit'`` the four masks
    are caller-supplied inputs (``set_masks``), with ``'philox'`` (default, the
    reference's behaviour) the kernels generate them from ``(seed, offset)``;
  * all intermediates of a pass live in ONE allocation (the reference makes
    23 + 27 ``torch.empty`` calls per iteration, pytorch_module/encoder.py:80-85,
    :110-121), and work is enqueued on the current torch stream;
  * ``activation='gelu'`` is available (the reference CUDA path is ReLU only).
There is no CPU path: tensors must be on a CUDA device.
"""

import ctypes
import os
import math

import torch

from . import _lib
from . import layouts as L

_ALIGN = 256


def _round_up(n, a=_ALIGN):
    return (n + a - 1) // a * a


# Replay of repeated passes as CUDA graphs inside the autograd path: off unless asked for.  The arenas, outputs
# and gradients of that path come from torch's caching allocator, whose blocks do not repeat reliably from step
# to step (measured: one capture per three steps, no gain), unlike the caller-held arenas of the raw passes.
_AUTOGRAD_GRAPHS = os.environ.get('SUBSTATION_B200_AUTOGRAD_GRAPHS', '0') == '1'

def _to_numpy(t):
    """numpy copy of a tensor for ``.debug``; numpy has no bfloat16, those come back as float32 (exact)."""
    t = t.detach()
    return (t.float() if t.dtype == torch.bfloat16 else t).cpu().numpy()


class Encoder(torch.nn.Module):
    """Optimized BERT encoder layer (API of pytorch_module/encoder.py:19-25)."""

    def __init__(self, compilation_dir, batch_size, max_seq_len, num_heads, embedding_size,
                 layouts, torch_dtype,
                 softmax_dropout_probability, residual1_dropout_probability,
                 activation_dropout_probability, residual2_dropout_probability,
                 enable_debug=False, profiling=False, *,
                 activation='relu', mask_mode='philox', seed=0, fuse=True, keep_all_intermediates=None):
        super().__init__()
        # float16 or bfloat16 storage, float32 accumulation; anything else (the reference also builds float and
        # double, pytorch_module/encoder.py:13-17) raises NotImplementedError
        self._lib_key = _lib.dtype_key(torch_dtype)
        if activation not in ('relu', 'gelu'):
            raise ValueError('Unknown activation ' + str(activation))
        if mask_mode not in ('philox', 'explicit'):
            raise ValueError("mask_mode must be 'philox' or 'explicit'")
        if embedding_size % num_heads:
            raise ValueError('embedding_size must be a multiple of num_heads')

        self.compilation_dir = compilation_dir  # accepted for compatibility; nothing is compiled per configuration
        self.batch_size = batch_size
        self.max_seq_len = max_seq_len
        self.num_heads = num_heads
        self.embedding_size = embedding_size
        self.proj_size = self.embedding_size // self.num_heads
        self.intermediate_size = self.embedding_size * 4
        self.softmax_dropout_probability = softmax_dropout_probability
        self.residual1_dropout_probability = residual1_dropout_probability
        self.activation_dropout_probability = activation_dropout_probability
        self.residual2_dropout_probability = residual2_dropout_probability
        self.torch_dtype = torch_dtype
        self.debug = {}  # intermediate tensors as numpy arrays when enable_debug
        self.layouts = layouts
        self.enable_debug = enable_debug
        self.profiling = profiling
        self.activation = activation
        self.mask_mode = mask_mode
        self.seed = int(seed)
        self.fuse = bool(fuse)          # fused multi-operator kernels where layouts allow (False: one kernel per reference operator)
        # Nine intermediates are read by nothing once the fused operators run (BETA, WKKWQQWVV, SB1_LINW1, LIN2,
        # the bias written back over ATT, DATTN_DROP, DLN2, DLN1, DXATT).  They are still written when somebody
        # can look at them (enable_debug) or asks for it; otherwise the kernels skip those stores.
        self.keep_all_intermediates = bool(enable_debug) if keep_all_intermediates is None else bool(keep_all_intermediates)
        self.philox_offset = 0          # advanced by 4 per forward, one per dropout site
        self._masks = None
        self._handle = None
        self._handle_device = None

        self._table = L.validate(layouts)
        self.sizes = L.sizes_map(batch_size, max_seq_len, num_heads, embedding_size)

        # Parameters: one per entry of layouts['params'], shaped by its dim letters
        # (pytorch_module/encoder.py:56-60).
        for param, layout in layouts['params']:
            sz = L.shape_of(layout, self.sizes)
            setattr(self, param, torch.nn.Parameter(torch.empty(*sz, dtype=self.torch_dtype)))
        self.params = tuple(getattr(self, k) for k, _ in layouts['params'])
        self.reset_parameters()

        self._fwd_names = [n for n, _ in layouts['forward_interm']]
        self._bwd_names = [n for n, _ in layouts['backward_interm']]
        self._param_names = [n for n, _ in layouts['params']]
        self._fwd_plan = self._plan(layouts['forward_interm'])
        self._bwd_plan = self._plan(layouts['backward_interm'])
        self._grad_plan = self._plan(layouts['params'])
        # (shape, contiguous strides, element offset) of each parameter gradient inside the gradient arena
        self._grad_views = []
        for _, shape, _, off, _ in self._grad_plan[0]:
            strides, acc = [], 1
            for extent in reversed(shape):
                strides.append(acc)
                acc *= extent
            self._grad_views.append((tuple(shape), tuple(reversed(strides)), off // 2))

        outer = self

        class EncoderFunction(torch.autograd.Function):
            @staticmethod
            def forward(ctx, X, anchor, *weights):
                # Hot path: one arena per pass, pointers computed from the plan's offsets; tensor views
                # over the arena are only built when somebody asks for them (debug, or a caller of views()).
                # ``anchor`` is None on the ordinary path (``weights`` are the sixteen parameters, and autograd routes
                # their gradients).  With a buffer pool it is a one-element leaf that keeps the node in the graph,
                # ``weights`` is ONE tuple of detached parameters that autograd does not look into, and backward
                # writes every ``.grad`` itself: sixteen inputs and sixteen accumulation nodes less per step.
                ctx.direct = anchor is not None
                if ctx.direct:
                    weights = weights[0]
                outer._check_input(X, 'X')
                X = X.contiguous()
                weights = tuple(w if w.is_contiguous() else w.contiguous() for w in weights)
                plan, total = outer._fwd_plan
                pooled = outer._pool_set(X) if outer.__dict__.get('_pool_n') else None
                if pooled is not None:
                    Y, arena = pooled['Y'], pooled['fwd']
                    ctx.pool_set = pooled
                else:
                    Y = torch.empty_like(X)
                    arena = torch.empty(max(total, 1), dtype=torch.uint8, device=X.device)
                    ctx.pool_set = None
                over = outer._explicit_masks(X.device) if outer.mask_mode == 'explicit' else {}
                ptrs = outer._pooled_ptrs('fwd', plan, arena, over) if pooled is not None else \
                    outer._plan_ptrs(plan, arena, over)
                outer._forward_ptrs(X, weights, ptrs, Y)
                if ctx.direct:
                    ctx.weights = weights
                    ctx.save_for_backward(arena, X)
                else:
                    ctx.save_for_backward(*weights, arena, X)
                ctx.masks = over
                if outer.enable_debug:
                    torch.cuda.synchronize()
                    fwd = outer.views('forward', arena)
                    fwd.update(over)
                    for name in outer._fwd_names:
                        outer.debug[name] = _to_numpy(fwd[name])
                    for name, w in zip(outer._param_names, weights):
                        outer.debug[name] = _to_numpy(w)
                return Y

            @staticmethod
            def backward(ctx, DY):
                saved = ctx.saved_tensors
                np_ = len(outer._param_names)
                if ctx.direct:
                    weights, arena, X = ctx.weights, saved[0], saved[1]
                else:
                    weights, arena, X = saved[:np_], saved[np_], saved[-1]
                outer._check_input(DY, 'DY')
                DY = DY.contiguous()
                bplan, btotal = outer._bwd_plan
                gplan, gtotal = outer._grad_plan
                if ctx.pool_set is not None:
                    DX, barena = ctx.pool_set['DX'], ctx.pool_set['bwd']
                    garena = ctx.pool_set['grads'] if not outer.__dict__.get('_grad_arenas') else \
                        outer._next_grad_arena(gtotal, DY.device)
                else:
                    DX = torch.empty_like(DY)
                    barena = torch.empty(max(btotal, 1), dtype=torch.uint8, device=DY.device)
                    garena = outer._next_grad_arena(gtotal, DY.device)
                tab = outer._pooled_ptrs if ctx.pool_set is not None else \
                    (lambda which, plan, a, over: outer._plan_ptrs(plan, a, over))
                outer._backward_ptrs(DY, tab('grads', gplan, garena, {}), tab('bwd', bplan, barena, {}), weights,
                                     tab('fwd', outer._fwd_plan[0], arena, ctx.masks), X, DX)
                g16 = garena[:max(gtotal, 2)].view(outer.torch_dtype)
                outer._grad_bucket = g16
                grads = tuple(torch.as_strided(g16, shape, strides, off) for shape, strides, off in outer._grad_views)
                if outer.enable_debug:
                    torch.cuda.synchronize()
                    bwd = outer.views('backward', barena)
                    for name in outer._bwd_names:
                        outer.debug[name] = _to_numpy(bwd[name])
                    for name, g in zip(outer._param_names, grads):
                        outer.debug['D' + name] = _to_numpy(g)
                if ctx.direct:
                    for prm, g in zip(outer.params, grads):
                        if prm.requires_grad:
                            prm.grad = g
                    return DX, None, None
                return (DX, None, *grads)

        self.encoder_func = EncoderFunction

    # ------------------------------------------------------------------ parameters
    def reset_parameters(self):
        """uniform(-1/sqrt(2), 1/sqrt(2)) as in pytorch_module/encoder.py:144-158."""
        stdev = 1.0 / math.sqrt(2)
        for weight in self.parameters():
            t = torch.empty_like(weight, dtype=torch.float32)
            torch.nn.init.uniform_(t, -stdev, stdev)
            with torch.no_grad():
                weight[:] = t

    # ------------------------------------------------------------------ buffers
    def _plan(self, entries):
        """(name, shape, dtype, byte offset) for one arena holding all listed tensors."""
        plan, off = [], 0
        for name, layout in entries:
            shape = L.shape_of(layout, self.sizes)
            dtype = torch.uint8 if name in L.MASKS else self.torch_dtype
            nbytes = math.prod(shape) * (1 if dtype == torch.uint8 else 2)
            plan.append((name, shape, dtype, off, nbytes))
            off += _round_up(nbytes)
        return plan, off

    @staticmethod
    def _alloc(plan_total, device):
        plan, total = plan_total
        arena = torch.empty(max(total, 1), dtype=torch.uint8, device=device)
        out = {}
        for name, shape, dtype, off, nbytes in plan:
            out[name] = arena[off:off + nbytes].view(dtype).view(shape)
        out['__arena__'] = arena
        return out

    def views(self, which, arena):
        """Named tensor views over a caller-provided uint8 arena; ``which`` is 'forward',
        'backward' or 'grads'.  Lets a caller keep buffers alive across steps (or place the
        gradients inside a communication bucket) instead of allocating per pass."""
        plan, total = {'forward': self._fwd_plan, 'backward': self._bwd_plan, 'grads': self._grad_plan}[which]
        if arena.dtype != torch.uint8 or arena.numel() < total or not arena.is_contiguous():
            raise ValueError(f'arena must be a contiguous uint8 tensor of at least {total} bytes')
        out = {}
        for name, shape, dtype, off, nbytes in plan:
            out[name] = arena[off:off + nbytes].view(dtype).view(shape)
        out['__arena__'] = arena
        return out

    def arena_bytes(self, which):
        return {'forward': self._fwd_plan, 'backward': self._bwd_plan, 'grads': self._grad_plan}[which][1]

    def intermediate_bytes(self):
        """Bytes of the forward and backward arenas (what one layer keeps alive)."""
        return self._fwd_plan[1], self._bwd_plan[1]

    def set_masks(self, masks):
        """Dropout masks for ``mask_mode='explicit'``: dict with ATTN_DROP_MASK,
        DROP1MASK, DROP2MASK, DROP3MASK -> uint8 {0,1} tensors stored in the layout
        the configuration gives each mask.  They are used in place (no copy)."""
        if masks is not None:
            for name in L.MASKS:
                if name not in masks:
                    raise KeyError(f'missing mask {name}')
                t = masks[name]
                want = L.shape_of(self._table[name], self.sizes)
                if t.dtype != torch.uint8 or tuple(t.shape) != want or not t.is_contiguous():
                    raise ValueError(f'mask {name} must be a contiguous uint8 tensor of shape {want}')
        self._masks = masks

    def _explicit_masks(self, device):
        if self._masks is None:
            raise RuntimeError("mask_mode='explicit' needs set_masks(...) before forward")
        for t in self._masks.values():
            if t.device != device:
                raise ValueError('masks must live on the same device as the input')
        return {n: self._masks[n] for n in L.MASKS}

    # ------------------------------------------------------------------ native handle
    def _native(self, device):
        if self._handle is not None and self._handle_device == device:
            return self._handle
        if self._handle is not None:
            self._destroy()
        lib = _lib.load(self._lib_key)
        names = list(self._table.keys())
        cfg = _lib.SbEncoderConfig()
        cfg.batch, cfg.seq = self.batch_size, self.max_seq_len
        cfg.heads, cfg.embed = self.num_heads, self.embedding_size
        cfg.activation = _lib.SB_ACT_RELU if self.activation == 'relu' else _lib.SB_ACT_GELU
        cfg.p_softmax = self.softmax_dropout_probability
        cfg.p_resid1 = self.residual1_dropout_probability
        cfg.p_activation = self.activation_dropout_probability
        cfg.p_resid2 = self.residual2_dropout_probability
        # pointer-table order = order of the configuration's lists (pytorch_module/encoder.py:229-299)
        ordered = (['X', 'SB2'] + self._param_names + self._fwd_names + self._bwd_names)
        assert sorted(ordered) == sorted(names)
        cfg.n_tensors = len(ordered)
        name_arr = (ctypes.c_char_p * len(ordered))(*[n.encode() for n in ordered])
        dims_arr = (ctypes.c_char_p * len(ordered))(*[self._table[n].encode() for n in ordered])
        cfg.names, cfg.dims = name_arr, dims_arr
        handle = ctypes.c_void_p()
        with torch.cuda.device(device):
            self._check(lib.sb_encoder_create(ctypes.byref(cfg), ctypes.byref(handle)))
            if self.profiling:
                self._check(lib.sb_encoder_set_timing(handle, 1))
            self._check(lib.sb_encoder_set_fusion(handle, 1 if self.fuse else 0))
            self._check(lib.sb_encoder_set_dead_stores(handle, 1 if self.keep_all_intermediates else 0))
            self._graphs_state = None
        self._handle, self._handle_device = handle, device
        with torch.cuda.device(device):
            self._apply_ffn_event()
        return handle

    def _check(self, status):
        _lib.check(status, _lib.load(self._lib_key))

    def _destroy(self):
        if self.__dict__.get('_handle') is not None:
            try:
                _lib.load(self._lib_key).sb_encoder_destroy(self._handle)
            except Exception:  # interpreter shutdown
                pass
            self._handle = None

    def __del__(self):
        self._destroy()

    @staticmethod
    def _ptrs(tensors):
        arr = (ctypes.c_void_p * len(tensors))()
        for i, t in enumerate(tensors):
            arr[i] = t.data_ptr()
        return arr

    def _check_input(self, X, what):
        want = L.shape_of(self._table['X'], self.sizes)
        if not X.is_cuda:
            raise ValueError(f'{what} must be a CUDA tensor (there is no CPU path)')
        if X.dtype != self.torch_dtype or tuple(X.shape) != want:
            raise ValueError(f'{what} must be {self.torch_dtype} of shape {want} '
                             f'(layout {self._table["X"]}), got {X.dtype} {tuple(X.shape)}')

    # ------------------------------------------------------------------ pointer-level passes
    @staticmethod
    def _plan_ptrs(plan, arena, overrides):
        """Device pointers of a plan's tensors inside ``arena`` (plan order); ``overrides``: name ->
        tensor that lives elsewhere (the caller's explicit masks)."""
        base = arena.data_ptr()
        arr = (ctypes.c_void_p * len(plan))()
        for i, (name, _, _, off, _) in enumerate(plan):
            t = overrides.get(name) if overrides else None
            arr[i] = base + off if t is None else t.data_ptr()
        return arr

    def _pooled_ptrs(self, which, plan, arena, overrides):
        """``_plan_ptrs`` remembered per (plan, arena, override pointers): with a buffer pool the same few arenas
        come back every step, and building a 50-entry pointer table three times per step is host time the
        end-to-end path can do without."""
        cache = self.__dict__.setdefault('_ptr_cache', {})
        key = (which, arena.data_ptr(), tuple(t.data_ptr() for t in overrides.values()) if overrides else ())
        arr = cache.get(key)
        if arr is None:
            if len(cache) > 64:
                cache.clear()
            arr = cache[key] = self._plan_ptrs(plan, arena, overrides)
        return arr

    def _graphs_now(self, h, on):
        """Graph replay pays when the buffers of a pass repeat (raw passes into caller-held arenas); the autograd
        path allocates fresh arenas per step, where capturing would only cost host time."""
        on = bool(on and self.__dict__.get('_graphs', True))
        if self.__dict__.get('_graphs_state') != on:
            self._check(_lib.load(self._lib_key).sb_encoder_set_graphs(h, int(on)))
            self._graphs_state = on

    def _forward_ptrs(self, X, weights, fwd_ptrs, Y):
        lib = _lib.load(self._lib_key)
        h = self._native(X.device)
        self._graphs_now(h, _AUTOGRAD_GRAPHS or bool(self.__dict__.get('_pool_n')))
        mode = _lib.SB_MASK_PHILOX if self.mask_mode == 'philox' else _lib.SB_MASK_EXPLICIT
        stream = ctypes.c_void_p(torch.cuda.current_stream(X.device).cuda_stream)
        self._check(lib.sb_encoder_forward(h, stream, ctypes.c_void_p(X.data_ptr()), self._ptrs(weights), fwd_ptrs,
                                          ctypes.c_void_p(Y.data_ptr()), mode, self.seed, self.philox_offset))
        self.philox_offset += 4

    def _backward_ptrs(self, DY, grad_ptrs, bwd_ptrs, weights, fwd_ptrs, X, DX):
        lib = _lib.load(self._lib_key)
        h = self._native(DY.device)
        self._graphs_now(h, _AUTOGRAD_GRAPHS or bool(self.__dict__.get('_pool_n')))
        stream = ctypes.c_void_p(torch.cuda.current_stream(DY.device).cuda_stream)
        self._check(lib.sb_encoder_backward(h, stream, ctypes.c_void_p(DY.data_ptr()), grad_ptrs, bwd_ptrs,
                                           self._ptrs(weights), fwd_ptrs, ctypes.c_void_p(X.data_ptr()),
                                           ctypes.c_void_p(DX.data_ptr())))

    # ------------------------------------------------------------------ raw passes (no autograd)
    @staticmethod
    def _check_raw(device, **named):
        """The raw passes hand bare pointers to the library: every buffer must be dense and on the handle's
        device.  Nothing is copied silently (a copy would also change the pointers the graph cache keys on)."""
        for what, t in named.items():
            if isinstance(t, dict):
                Encoder._check_raw(device, **{f'{what}[{k}]': v for k, v in t.items() if k != '__arena__'})
            elif isinstance(t, (list, tuple)):
                Encoder._check_raw(device, **{f'{what}[{i}]': v for i, v in enumerate(t)})
            else:
                if t.device != device:
                    raise ValueError(f'{what} lives on {t.device}, the pass runs on {device}')
                if not t.is_contiguous():
                    raise ValueError(f'{what} must be contiguous (the raw passes take pointers, not views)')

    def forward_raw(self, X, weights, fwd, Y):
        """One forward pass into caller-provided buffers.  ``fwd``: name -> tensor for
        the 23 forward intermediates (see ``_alloc``).  All buffers contiguous, on one device."""
        self._check_input(X, 'X')
        self._check_input(Y, 'Y')
        self._check_raw(X.device, X=X, Y=Y, weights=list(weights), fwd={n: fwd[n] for n in self._fwd_names})
        lib = _lib.load(self._lib_key)
        h = self._native(X.device)
        self._graphs_now(h, True)
        mode = _lib.SB_MASK_PHILOX if self.mask_mode == 'philox' else _lib.SB_MASK_EXPLICIT
        stream = ctypes.c_void_p(torch.cuda.current_stream(X.device).cuda_stream)
        wl = list(weights)
        self._check(lib.sb_encoder_forward(
            h, stream, ctypes.c_void_p(X.data_ptr()), self._ptrs(wl),
            self._ptrs([fwd[n] for n in self._fwd_names]), ctypes.c_void_p(Y.data_ptr()),
            mode, self.seed, self.philox_offset))
        self.philox_offset += 4
        return Y

    def backward_raw(self, DY, grads, bwd, weights, fwd, X, DX):
        """One backward pass; ``grads``/``bwd``: name -> preallocated tensor."""
        self._check_input(DY, 'DY')
        self._check_input(DX, 'DX')
        self._check_input(X, 'X')
        self._check_raw(DY.device, DY=DY, DX=DX, X=X, weights=list(weights),
                        grads={n: grads[n] for n in self._param_names}, bwd={n: bwd[n] for n in self._bwd_names},
                        fwd={n: fwd[n] for n in self._fwd_names})
        lib = _lib.load(self._lib_key)
        h = self._native(DY.device)
        self._graphs_now(h, True)
        stream = ctypes.c_void_p(torch.cuda.current_stream(DY.device).cuda_stream)
        wl = list(weights)
        self._check(lib.sb_encoder_backward(
            h, stream, ctypes.c_void_p(DY.data_ptr()),
            self._ptrs([grads[n] for n in self._param_names]),
            self._ptrs([bwd[n] for n in self._bwd_names]),
            self._ptrs(wl), self._ptrs([fwd[n] for n in self._fwd_names]),
            ctypes.c_void_p(X.data_ptr()), ctypes.c_void_p(DX.data_ptr())))
        return DX

    def op_times(self):
        """[(operator name, ms)] of the passes since the last call (needs profiling=True).
        Names follow the NVTX ranges of pytorch_module/encoder.cu:89-296."""
        if self._handle is None:
            return []
        lib = _lib.load(self._lib_key)
        n = 64
        names = (ctypes.c_char_p * n)()
        ms = (ctypes.c_float * n)()
        k = lib.sb_encoder_get_timing(self._handle, n, names, ms)
        return [(names[i].decode(), ms[i]) for i in range(k)]

    # parameters whose gradients are final before the attention half of the backward pass runs
    _EARLY_GRADS = frozenset(('LINW1', 'LINB1', 'LINW2', 'LINB2', 'S1', 'B1', 'S2', 'B2', 'BO'))

    def early_grad_offset(self):
        """Byte offset in the gradient arena from which on every gradient belongs to the feed-forward half or a
        LayerNorm (final when the event of ``set_ffn_grads_event`` fires); equals the arena size if the
        configuration's parameter order ends with an attention parameter."""
        plan, total = self._grad_plan
        off = total
        for name, _, _, o, _ in reversed(plan):
            if name not in self._EARLY_GRADS:
                break
            off = o
        return off

    def set_ffn_grads_event(self, event):
        """``event``: a torch.cuda.Event that every backward pass records once those gradients are final, or None.
        A data-parallel caller waits for it on its communication stream (see GradientBucketReducer.reduce_async)."""
        self._ffn_event = event
        if self._handle is not None:
            self._apply_ffn_event()

    def _apply_ffn_event(self):
        ev = self.__dict__.get('_ffn_event')
        handle = None
        if ev is not None:
            if not ev.cuda_event:      # created lazily: a first record makes the handle exist
                ev.record()
            handle = ctypes.c_void_p(ev.cuda_event)
        self._check(_lib.load(self._lib_key).sb_encoder_set_ffn_grads_event(self._handle, handle))

    def set_buffer_pool(self, n, direct_grads=True):
        """``n`` > 0: the autograd path stops allocating per pass and takes the forward arena, the output, the backward
        arena, the input gradient and the gradient bucket from ``n`` sets of buffers the module owns, used in turn
        (allocated on first use).  The pointers of a pass then repeat every ``n`` steps, so passes are replayed as
        CUDA graphs with one launch each instead of some thirty, which is what an input pipeline that feeds the
        module from a few rotating device buffers wants.  The price: a tensor returned by ``forward`` (or a
        gradient produced by ``backward``) is overwritten ``n`` steps later; copy what must live longer.
        ``direct_grads``: backward sets every parameter's ``.grad`` itself (a view into the pooled bucket, replacing
        what was there) instead of handing sixteen gradients to autograd, which takes a third off the host's time per
        step; parameter hooks do not fire and ``torch.autograd.grad`` with respect to a parameter is not available
        on that path (pass ``direct_grads=False`` to keep autograd's routing).  ``n`` = 0 (the default) restores the
        reference's behaviour, fresh tensors every pass (pytorch_module/encoder.py:80-85, :110-121)."""
        self._pool_direct = bool(direct_grads)
        self._pool_n = int(n)
        self._pool = []
        self._pool_turn = 0
        self._ptr_cache = {}

    def _pool_set(self, X):
        if len(self._pool) < self._pool_n:
            dev = X.device
            self._pool.append({
                'Y': torch.empty_like(X), 'DX': torch.empty_like(X),
                'fwd': torch.empty(max(self._fwd_plan[1], 1), dtype=torch.uint8, device=dev),
                'bwd': torch.empty(max(self._bwd_plan[1], 1), dtype=torch.uint8, device=dev),
                'grads': torch.empty(max(self._grad_plan[1], 2), dtype=torch.uint8, device=dev)})
            return self._pool[-1]
        s = self._pool[self._pool_turn % self._pool_n]
        self._pool_turn += 1
        if s['Y'].device != X.device:
            raise ValueError('the buffer pool lives on another device than the input; call set_buffer_pool again')
        return s

    def set_grad_arenas(self, arenas):
        """Caller-held storage for the parameter gradients of the autograd path: a list of contiguous uint8 CUDA
        tensors of at least ``arena_bytes('grads')`` bytes, used in turn by successive backward passes (``None``:
        back to a fresh allocation per pass).  A data-parallel caller that reduces ``grad_bucket()`` every step
        then hands the collective the same few buffers again and again; with two arenas the reduction of one
        step may still run while the next backward fills the other.  The caller must not let a backward pass
        start on an arena whose reduction is still in flight."""
        if arenas is not None:
            need = self.arena_bytes('grads')
            for a in arenas:
                if a.dtype != torch.uint8 or not a.is_contiguous() or a.numel() < need or not a.is_cuda:
                    raise ValueError(f'gradient arenas must be contiguous uint8 CUDA tensors of at least {need} bytes')
            arenas = list(arenas)
        self._grad_arenas = arenas
        self._grad_arena_turn = 0

    def _next_grad_arena(self, total, device):
        arenas = self.__dict__.get('_grad_arenas')
        if not arenas:
            return torch.empty(max(total, 1), dtype=torch.uint8, device=device)
        a = arenas[self._grad_arena_turn % len(arenas)]
        self._grad_arena_turn += 1
        if a.device != device:
            raise ValueError('gradient arenas must live on the device the pass runs on')
        return a

    def grad_bucket(self):
        """The flat fp16 tensor that holds all 12 parameter gradients of the most recent autograd backward
        (each ``.grad`` is a view into it): a data-parallel caller sums one tensor instead of twelve."""
        return self.__dict__.get('_grad_bucket')

    def set_graphs(self, enabled):
        """Replay passes whose buffers repeat as CUDA graphs (default) or launch every kernel each time."""
        self._graphs = bool(enabled)
        self._graphs_state = None

    def graph_stats(self):
        """(passes captured as CUDA graphs, passes replayed) since the native handle was created."""
        if self._handle is None:
            return 0, 0
        c, r = ctypes.c_longlong(0), ctypes.c_longlong(0)
        self._check(_lib.load(self._lib_key).sb_encoder_graph_stats(self._handle, ctypes.byref(c), ctypes.byref(r)))
        return c.value, r.value

    def launch_count(self):
        """Operators launched by the most recent raw pass."""
        return 0 if self._handle is None else _lib.load(self._lib_key).sb_encoder_launch_count(self._handle)

    def kernel_count(self):
        """Kernels launched by the most recent forward plus the most recent backward."""
        return 0 if self._handle is None else _lib.load(self._lib_key).sb_encoder_kernel_count(self._handle)

    def forward(self, X):
        """Run the encoder."""
        if self.__dict__.get('_pool_n') and self.__dict__.get('_pool_direct') and torch.is_grad_enabled():
            anchor = self.__dict__.get('_anchor')
            if anchor is None or anchor.device != X.device:
                anchor = self._anchor = torch.zeros(1, device=X.device, requires_grad=True)
            return self.encoder_func.apply(X, anchor, tuple(p.detach() for p in self.params))
        return self.encoder_func.apply(X, None, *self.params)
