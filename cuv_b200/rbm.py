"""The sparse-RBM contrastive-divergence (CD-1) step that calls the DIA path.

Call order and scaling follow CUV's RBM trainer (examples/rbm/base.py:223-258 with one Gibbs step;
upPass/downPass :48-54, gradient accumulation :76-83), with the dense weight products replaced by
their DIA forms.  W is hidden x visible, so the up pass is ``prod(..., 'n')`` and the down pass the
transposed product:

    H0p = sigm(W V0 + c)      H0 = H0p > U_h          prod 'n'  + bias/sigmoid/compare
    V1p = sigm(W^T H0 + b)    V1 = V1p > U_v          prod 't'  + bias/sigmoid/compare
    H1p = sigm(W V1 + c)                              prod 'n'  + bias/sigmoid
    G   =  (1/B) (H0p V0^T)|dia                       densedense_to_dia(factAB= 1/B, factC=0)
    G   = -(1/B) (H1p V1^T)|dia + G                   densedense_to_dia(factAB=-1/B, factC=1)
    gc  = (1/B)(sum_b H0p - sum_b H1p)                reduce_to_col x2 (second accumulates)
    gb  = (1/B)(sum_b V0  - sum_b V1)                 reduce_to_col x2

The uniform numbers U_h, U_v are inputs, so a step is deterministic.  With several ranks every rank
holds the batch columns ``[r*B/P, (r+1)*B/P)`` and its own copy of W; B in the factors is the global
batch, so the per-rank G, gc, gb are partial sums that one all-reduce completes.
"""
import cuv_b200 as cb


class SparseRBMStep:
    """One rank's CD-1 step.  ``step()`` is a single call of the C ABI (``cuvdia_rbm_cd1_step_f32``); ``forward()`` +
    ``gradients()`` issue the same kernels call by call (used when the calls are timed one by one, or when the inputs
    arrive while the step runs).

    ``bias_sums="glue"`` (default): the bias gradients come from the element-wise passes that already stream H0p, V1
    and H1p, and only the sum over V0 is a reduction of its own.  ``"reduce"``: four ``reduce_to_col`` calls after
    the products, as the trainer issues them (examples/rbm/base.py:76-83); ``fused=True`` additionally calls the
    combined product + bias/logistic/compare entry point.  ``keep_v1p=False`` does not write the reconstruction's
    probabilities back (only its sample is used afterwards)."""

    def __init__(self, W, batch_local, batch_global=None, mode=cb.MODE_EXACT, device="cuda", fused=False,
                 bias_sums="glue", keep_v1p=True):
        import torch
        self.W = W
        self.hid, self.vis = W.h, W.w
        self.nb = int(batch_local)
        self.B = int(batch_global if batch_global is not None else batch_local)
        self.mode = mode
        self.fused = fused        # call the combined product + bias/logistic/compare entry point (same bits)
        self.bias_sums = "reduce" if fused else bias_sums
        self.keep_v1p = keep_v1p
        self.dev = device
        E = cb.colmajor_empty
        self.H0p, self.H0 = E(self.hid, self.nb, device), E(self.hid, self.nb, device)
        self.V1p, self.V1 = E(self.vis, self.nb, device), E(self.vis, self.nb, device)
        self.H1p = E(self.hid, self.nb, device)
        # gradient with W's layout; padding cells are never written, keep them at zero.  The diagonals' values and
        # the two bias gradients (gc, then gb) share one buffer so that a single collective covers them all.
        self.G = cb.dev_dia_matrix_f(W.h, W.w, W.offsets, W.stride, W.row_fact, device=device)
        n_g = self.G.vec.numel()
        if n_g % 4 == 0:
            self.grad_buf = torch.zeros(n_g + self.hid + self.vis, dtype=torch.float32, device=device)
            self.G.vec = self.grad_buf[:n_g]
            self.bias_grad = self.grad_buf[n_g:]
        else:
            self.grad_buf = None
            self.G.vec.zero_()
            self.bias_grad = torch.zeros(self.hid + self.vis, dtype=torch.float32, device=device)
        self.Gbd = cb.dev_block_descriptor_f(self.G)
        self.gc, self.gb = self.bias_grad[:self.hid], self.bias_grad[self.hid:]
        self.b_vis = torch.zeros(self.vis, dtype=torch.float32, device=device)
        self.c_hid = torch.zeros(self.hid, dtype=torch.float32, device=device)
        self.timers = None        # optional dict name -> list of (start_event, end_event)
        self._reducer = None

    def _timed(self, name, fn):
        if self.timers is None:
            return fn()
        import torch
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        r = fn()
        e1.record()
        self.timers.setdefault(name, []).append((e0, e1))
        return r

    def step(self, V0, U_h, U_v):
        """One CD-1 gradient evaluation on this rank's batch columns; results in G.vec, gc, gb
        (partial sums when batch_global > batch_local)."""
        if self.timers is None and self.bias_sums == "glue":
            return self._step_c(V0, U_h, U_v)
        self.forward(V0, U_h, U_v)
        self.gradients(V0)

    def step_allreduce(self, V0, U_h, U_v, group=None, overlap=1):
        """step() followed by allreduce() as one call of the C ABI (``cuvdia_rbm_cd1_step_allreduce_f32``): the
        all-reduce of the diagonals that the step's last kernel completes first runs while that kernel finishes the
        rest.  Same results as the two separate calls.  ``overlap``: 0 never, 1 when cutting the kernel's grid in two
        costs no wave of blocks, 2 whenever the tiled kernel applies."""
        if self._reducer is None:
            self._reducer = GradientAllReduce(self.dev, group)
        if self.timers is not None or self.bias_sums != "glue":
            self.step(V0, U_h, U_v)
            return self.allreduce(group)
        self._step_c(V0, U_h, U_v, comm=self._reducer.comm, overlap=overlap)

    def step_drawn(self, V0, seed, step=0, col0=0):
        """step() with the uniform numbers of the two samples drawn on the device (``cuvdia_rbm_cd1_step_drawn_f32``):
        the bits of ``step(V0, U_h, U_v)`` on ``U_h = cb.fill_rnd_uniform(.., which=0)`` and ``U_v = .. which=1`` with
        the same ``seed``, ``step`` and ``col0`` (global index of this rank's first batch column).  Nothing but V0 has
        to reach the device."""
        return self._step_c(V0, None, None, draw=(seed, step, col0))

    def step_drawn_allreduce(self, V0, seed, step=0, col0=0, group=None, overlap=1):
        """step_drawn() and the all-reduce of the gradients as one call of the C ABI."""
        if self._reducer is None:
            self._reducer = GradientAllReduce(self.dev, group)
        return self._step_c(V0, None, None, comm=self._reducer.comm, overlap=overlap, draw=(seed, step, col0))

    def _step_c(self, V0, U_h, U_v, comm=None, overlap=1, draw=None):
        """The whole step as one call of the C ABI."""
        import ctypes
        from . import _capi
        inputs = ((V0, self.vis, "V0"),) if draw is not None else ((V0, self.vis, "V0"), (U_h, self.hid, "U_h"), (U_v, self.vis, "U_v"))
        for t, rows, name in inputs:
            if cb._check_colmajor(t, name) != rows or t.shape != (rows, self.nb):
                raise cb.CuvDiaError(_capi.ERR_INVALID, name + " must be a dense column-major [units x batch] matrix")
        p = lambda t: t.data_ptr() if t is not None else None
        buf = _capi.RbmCd1Buffers(p(V0), p(U_h), p(U_v), p(self.b_vis), p(self.c_hid), p(self.H0p), p(self.H0),
                                  p(self.V1p), p(self.V1), p(self.H1p), p(self.G.vec), p(self.gc), p(self.gb))
        if draw is not None:
            d = _capi.Draw(int(draw[0]), int(draw[1]), int(draw[2]))
            if comm is not None:
                _capi.check(_capi.lib().cuvdia_rbm_cd1_step_drawn_allreduce_f32(
                    self.W._plan, cb._ptr(self.W.vec), ctypes.byref(buf), self.nb, self.B, self.mode,
                    1 if self.keep_v1p else 0, ctypes.byref(d), int(overlap), comm, cb._stream()))
            else:
                _capi.check(_capi.lib().cuvdia_rbm_cd1_step_drawn_f32(
                    self.W._plan, cb._ptr(self.W.vec), ctypes.byref(buf), self.nb, self.B, self.mode,
                    1 if self.keep_v1p else 0, ctypes.byref(d), cb._stream()))
            return
        if comm is not None:
            _capi.check(_capi.lib().cuvdia_rbm_cd1_step_allreduce_f32(
                self.W._plan, cb._ptr(self.W.vec), ctypes.byref(buf), self.nb, self.B, self.mode,
                1 if self.keep_v1p else 0, int(overlap), comm, cb._stream()))
            return
        _capi.check(_capi.lib().cuvdia_rbm_cd1_step_f32(self.W._plan, cb._ptr(self.W.vec), ctypes.byref(buf), self.nb,
                                                        self.B, self.mode, 1 if self.keep_v1p else 0, cb._stream()))

    def forward(self, V0, U_h, U_v, arrived=None, draw=None):
        """The three products with their bias/logistic/sampling passes (and, with ``bias_sums="glue"``, the bias
        gradients).  ``arrived``: optional events (V0, U_h, U_v) that the current stream waits for just before the
        first use of each input, so that a step can start on V0 while the uniform numbers are still on their way.
        ``draw=(seed, step, col0)``: the uniform numbers are drawn inside the element-wise passes (U_h, U_v unused)."""
        W = self.W
        t = self._timed
        inv = 1.0 / self.B

        def need(k):
            if arrived is not None:
                import torch
                torch.cuda.current_stream().wait_event(arrived[k])

        if self.fused:
            F = cb.prod_bias_sigmoid_sample
            need(0); need(1)
            t("prod_n", lambda: F(self.H0p, W, V0, "n", 1.0, 0.0, self.mode, self.c_hid, U_h, self.H0))
            need(2)
            t("prod_t", lambda: F(self.V1p, W, self.H0, "t", 1.0, 0.0, self.mode, self.b_vis, U_v, self.V1))
            t("prod_n", lambda: F(self.H1p, W, self.V1, "n", 1.0, 0.0, self.mode, self.c_hid))
            return
        need(0)
        if draw is not None:
            if self.bias_sums != "glue" or self.fused:
                raise ValueError("drawn samples come with the bias sums taken in the element-wise passes")
            GS, DS = cb.bias_sigmoid_sample_sum, cb.bias_sigmoid_draw_sum
            seed, stepno, col0 = draw
            t("reduce", lambda: cb.reduce_to_col(self.gb, V0, cb.RF_ADD, inv, 0.0))
            t("prod_n", lambda: cb.prod(self.H0p, W, V0, "n", "n", 1.0, 0.0, self.mode))
            t("glue", lambda: DS(self.H0p, self.c_hid, self.H0, self.gc, seed, stepno, col0, 0, False, inv, 0.0))
            t("prod_t", lambda: cb.prod(self.V1p, W, self.H0, "t", "n", 1.0, 0.0, self.mode))
            t("glue", lambda: DS(self.V1p, self.b_vis, self.V1, self.gb, seed, stepno, col0, 1, True, -inv, 1.0,
                                 self.keep_v1p))
            t("prod_n", lambda: cb.prod(self.H1p, W, self.V1, "n", "n", 1.0, 0.0, self.mode))
            t("glue", lambda: GS(self.H1p, self.c_hid, None, None, self.gc, False, -inv, 1.0))
            return
        if self.bias_sums == "glue":
            GS = cb.bias_sigmoid_sample_sum
            t("reduce", lambda: cb.reduce_to_col(self.gb, V0, cb.RF_ADD, inv, 0.0))
            t("prod_n", lambda: cb.prod(self.H0p, W, V0, "n", "n", 1.0, 0.0, self.mode))
            need(1)
            t("glue", lambda: GS(self.H0p, self.c_hid, U_h, self.H0, self.gc, False, inv, 0.0))
            t("prod_t", lambda: cb.prod(self.V1p, W, self.H0, "t", "n", 1.0, 0.0, self.mode))
            need(2)
            t("glue", lambda: GS(self.V1p, self.b_vis, U_v, self.V1, self.gb, True, -inv, 1.0, self.keep_v1p))
            t("prod_n", lambda: cb.prod(self.H1p, W, self.V1, "n", "n", 1.0, 0.0, self.mode))
            t("glue", lambda: GS(self.H1p, self.c_hid, None, None, self.gc, False, -inv, 1.0))
            return
        t("prod_n", lambda: cb.prod(self.H0p, W, V0, "n", "n", 1.0, 0.0, self.mode))
        need(1)
        t("glue", lambda: cb.bias_sigmoid_sample(self.H0p, self.c_hid, U_h, self.H0))
        t("prod_t", lambda: cb.prod(self.V1p, W, self.H0, "t", "n", 1.0, 0.0, self.mode))
        need(2)
        t("glue", lambda: cb.bias_sigmoid_sample(self.V1p, self.b_vis, U_v, self.V1))
        t("prod_n", lambda: cb.prod(self.H1p, W, self.V1, "n", "n", 1.0, 0.0, self.mode))
        t("glue", lambda: cb.bias_sigmoid_sample(self.H1p, self.c_hid))

    def gradients(self, V0):
        """Weight-gradient diagonals (and, with ``bias_sums="reduce"``, the bias gradients) from the activations of
        forward()."""
        inv = 1.0 / self.B
        t = self._timed
        t("dd2dia", lambda: cb.densedense_to_dia(self.G, self.Gbd, self.H0p, V0, inv, 0.0))
        t("dd2dia", lambda: cb.densedense_to_dia(self.G, self.Gbd, self.H1p, self.V1, -inv, 1.0))
        if self.bias_sums == "glue":
            return
        t("reduce", lambda: cb.reduce_to_col(self.gc, self.H0p, cb.RF_ADD, inv, 0.0))
        t("reduce", lambda: cb.reduce_to_col(self.gc, self.H1p, cb.RF_ADD, -inv, 1.0))
        t("reduce", lambda: cb.reduce_to_col(self.gb, V0, cb.RF_ADD, inv, 0.0))
        t("reduce", lambda: cb.reduce_to_col(self.gb, self.V1, cb.RF_ADD, -inv, 1.0))

    def allreduce(self, group=None):
        """Sum the partial gradients over the ranks (NCCL over NVLink): the diagonals of G and the two bias
        gradients, one collective issued through the C ABI on a communicator of the library's own."""
        if self._reducer is None:
            self._reducer = GradientAllReduce(self.dev, group)
        self._reducer(self.G.vec, self.bias_grad)

    def capture(self, V0, U_h, U_v):
        """Records one step on the given (static) input tensors into a CUDA graph and returns it; ``graph.replay()``
        then runs the kernels of a step with a single launch.  The library allocates its scratch buffers on first
        use, so one ordinary step is run first; nothing is allocated while recording."""
        import torch
        timers, self.timers = self.timers, None          # events cannot be recorded into the graph this way
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            self.step(V0, U_h, U_v)                      # on the recording stream: the reductions' workspace is per stream
            side.synchronize()
            with torch.cuda.graph(graph, stream=side):
                self.step(V0, U_h, U_v)
        torch.cuda.current_stream().wait_stream(side)
        self.timers = timers
        return graph

    def update(self, learnrate, decay=0.0):
        """The trainer's update step (examples/rbm/base.py:72-75): learn_step_weight_decay on the weight
        diagonals and on both bias vectors with the gradients of the last step (after allreduce() when
        there are several ranks, so that every rank applies the same full-batch gradient)."""
        t = self._timed
        t("update", lambda: cb.learn_step_weight_decay(self.W, self.G, learnrate, decay))
        t("update", lambda: cb.learn_step_weight_decay(self.c_hid, self.gc, learnrate, decay))
        t("update", lambda: cb.learn_step_weight_decay(self.b_vis, self.gb, learnrate, decay))


class GradientAllReduce:
    """In-place sum of the partial gradients over the ranks through ``cuvdia_allreduce_grad``.  The NCCL
    communicator is the library's own (``cuvdia_nccl_comm_create``): rank 0 draws the unique id and
    ``torch.distributed`` only carries its 128 bytes to the other ranks."""

    def __init__(self, device, group=None):
        import ctypes
        import torch
        import torch.distributed as dist
        from . import _capi
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        ident = torch.zeros(128, dtype=torch.uint8, device=device)
        if self.rank == 0:
            raw = ctypes.create_string_buffer(128)
            _capi.check(_capi.lib().cuvdia_nccl_unique_id(raw))
            ident.copy_(torch.frombuffer(bytearray(raw.raw), dtype=torch.uint8))
        src = dist.get_global_rank(group, 0) if group is not None else 0
        dist.broadcast(ident, src=src, group=group)
        self.comm = ctypes.c_void_p()
        with torch.cuda.device(torch.device(device)):
            _capi.check(_capi.lib().cuvdia_nccl_comm_create(ctypes.byref(self.comm), self.world, self.rank,
                                                            bytes(ident.cpu().numpy().tobytes())))

    def __call__(self, g_vec, bias_grad):
        from . import _capi
        _capi.check(_capi.lib().cuvdia_allreduce_grad(self.comm, cb._ptr(g_vec), g_vec.numel(), cb._ptr(bias_grad),
                                                      bias_grad.numel(), cb._stream()))

    def close(self):
        from . import _capi
        comm, self.comm = self.comm, None
        if comm:
            _capi.check(_capi.lib().cuvdia_nccl_comm_destroy(comm))


class HostFedRBM:
    """Runs SparseRBMStep on inputs that live in pinned host memory and returns the gradients to
    pinned host memory, with the transfers overlapped with compute: the host-to-device copies of step
    i+1 run on a copy stream while step i computes (two device input sets), a step starts as soon as
    its first input has arrived (the uniform numbers are awaited where they are first used), and the
    device-to-host read of step i's gradients runs on a third stream while step i+1's products
    compute."""

    def __init__(self, step, allreduce=False, draw=None):
        """``draw=(seed, col0)``: the uniform numbers are drawn on the device (step number = count of steps run), so
        only V0 is copied per step and ``submit`` takes one tensor."""
        import torch
        self.step, self.allreduce, self.draw = step, allreduce, draw
        dev = step.dev
        E = cb.colmajor_empty
        if draw is not None:
            self.inputs = [(E(step.vis, step.nb, dev),) for _ in range(2)]
        else:
            self.inputs = [(E(step.vis, step.nb, dev), E(step.hid, step.nb, dev), E(step.vis, step.nb, dev))
                           for _ in range(2)]
        self.h2d, self.d2h = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        self.ready = [[torch.cuda.Event() for _ in range(3)] for _ in range(2)]     # per slot: V0, U_h, U_v arrived
        self.consumed = [torch.cuda.Event() for _ in range(2)]
        self.grads_done, self.fetched, self.bias_fetched = torch.cuda.Event(), torch.cuda.Event(), torch.cuda.Event()
        self.n_sub = self.n_run = 0
        self._fetch_pending = False

    def submit(self, hV0, hU_h=None, hU_v=None):
        """Queue the copy of one step's inputs (pinned host tensors holding the column-major matrices,
        i.e. shape (batch, units) contiguous)."""
        import torch
        slot = self.n_sub % 2
        if self.n_sub >= 2:
            self.h2d.wait_event(self.consumed[slot])
        with torch.cuda.stream(self.h2d):
            for k, (dst, src) in enumerate(zip(self.inputs[slot], (hV0, hU_h, hU_v))):      # one tensor when drawn
                dst.t().copy_(src, non_blocking=True)
                self.ready[slot][k].record(self.h2d)
        self.n_sub += 1

    def run(self, hG=None, hbias=None, g_range=None):
        """Compute the oldest submitted step; if host buffers are given, queue the read-back of its
        gradients into them.  ``g_range=(lo, hi)``: hG receives only the values lo .. hi-1 of the diagonals' array -
        after the all-reduce every rank holds the whole gradient, so each rank can send its own share to the host over
        its own link (hbias may then be None on all ranks but one)."""
        import torch
        cur = torch.cuda.current_stream()
        slot = self.n_run % 2
        V0 = self.inputs[slot][0]
        if self._fetch_pending:
            cur.wait_event(self.bias_fetched)     # forward() writes the bias gradients: their (small) read-back goes first
        if self.draw is not None:
            self.step.forward(V0, None, None, arrived=self.ready[slot], draw=(self.draw[0], self.n_run, self.draw[1]))
        else:
            U_h, U_v = self.inputs[slot][1:]
            self.step.forward(V0, U_h, U_v, arrived=self.ready[slot])   # each input is awaited where it is first used
        if self._fetch_pending:
            cur.wait_event(self.fetched)          # the previous gradients must have left before they are overwritten
        self.step.gradients(V0)
        if self.allreduce:
            self.step.allreduce()
        self.consumed[slot].record(cur)
        self.n_run += 1
        if hG is not None:
            self.grads_done.record(cur)
            self.d2h.wait_event(self.grads_done)
            with torch.cuda.stream(self.d2h):
                if hbias is not None:
                    hbias.copy_(self.step.bias_grad, non_blocking=True)
                self.bias_fetched.record(self.d2h)
                src = self.step.G.vec if g_range is None else self.step.G.vec[g_range[0]:g_range[1]]
                hG[:src.numel()].copy_(src, non_blocking=True)
                self.fetched.record(self.d2h)
            self._fetch_pending = True

    def wait(self):
        import torch
        torch.cuda.current_stream().wait_stream(self.d2h)
        torch.cuda.current_stream().wait_stream(self.h2d)


def shard_columns(batch_global, world, rank):
    """Batch columns [c0, c1) that ``rank`` of ``world`` owns; the dense operands are column-major,
    so a shard is one contiguous block of memory."""
    if batch_global % world:
        raise ValueError("the global batch must divide evenly over the ranks")
    nb = batch_global // world
    return rank * nb, (rank + 1) * nb


def allreduce_gradients(g_vec, bias_grad, group=None):
    """In-place sum over the ranks of the per-rank partial gradients (every rank computed its
    partials with the GLOBAL batch in the 1/B factor, so the sum is the full-batch gradient) with
    ``torch.distributed``'s own collectives: the host-side ranks of the CPU tests (gloo) use this; on GPUs
    ``SparseRBMStep.allreduce`` goes through the C ABI instead."""
    import torch.distributed as dist
    dist.all_reduce(g_vec, op=dist.ReduceOp.SUM, group=group)
    dist.all_reduce(bias_grad, op=dist.ReduceOp.SUM, group=group)


def algorithmic_work(h, w, nd, nnz, nb):
    """Bytes and flops of one step on ``nb`` batch columns, each operand counted once per routine
    (prod: A values + offsets + B + C; densedense_to_dia: both dense operands + offsets + the
    diagonals once or twice; reduction: the matrix + the output once or twice)."""
    prod_n = 4 * (nnz + nd + w * nb + h * nb)
    prod_t = 4 * (nnz + nd + h * nb + w * nb)
    dd0 = 4 * (h * nb + w * nb + nd + nnz)
    dd1 = 4 * (h * nb + w * nb + nd + 2 * nnz)
    red = lambda n, acc: 4 * (n * nb + n * (2 if acc else 1))
    glue_s, glue_n = 4 * 4, 4 * 2        # bytes per element: act r/w + u + sample, or act r/w
    byts = {"prod_n": prod_n, "prod_t": prod_t, "dd2dia": (dd0 + dd1) / 2.0,
            "reduce": (red(h, 0) + red(h, 1) + red(w, 0) + red(w, 1)) / 4.0,
            "reduce_v0": red(w, 0),      # the one reduction left when the element-wise passes take the other sums
            "glue": (glue_s * h * nb + glue_s * w * nb + glue_n * h * nb) / 3.0}
    total_bytes = 2 * prod_n + prod_t + dd0 + dd1 + red(h, 0) + red(h, 1) + red(w, 0) + red(w, 1)
    flops = 5 * 2.0 * nnz * nb
    return {"bytes": float(total_bytes), "flops": flops, "per_call_bytes": byts,
            "per_call_flops": {"prod_n": 2.0 * nnz * nb, "prod_t": 2.0 * nnz * nb, "dd2dia": 2.0 * nnz * nb}}
