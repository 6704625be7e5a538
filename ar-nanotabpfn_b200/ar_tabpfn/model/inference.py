"""Autoregressive predictor with layout-fixed KV caches on sm_100a kernels.

Same class, method names, argument shapes and error behaviour as the reference
``ARTabPFNPredictor`` (ar_tabpfn/model/inference.py:32-890).  Both backend names
are accepted and select the context-sharing semantics, not an implementation:

  * ``"triton_shared_context"``: one context K/V (taken from batch element 0,
    like the reference, inference.py:191-193) shared by every sample stream;
  * ``"flex_attention"`` (default): every batch element keeps its own context.

All compute runs in libartab_b200.so; there is no Python or CPU fallback.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch
from torch import Tensor

from .. import _lib
from .._pack import packed_for


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


class ARTabPFNPredictor:
    """Joint sampling and log-density evaluation."""

    def __init__(self, embedder, backbone, head, ar_tokens, backend: str = "flex_attention",
                 precision: Optional[str] = None):
        """
        Args:
            embedder, backbone, head, ar_tokens: the four pieces of an ``ARTabPFN``.
            backend: "flex_attention" (per-batch context) or "triton_shared_context".
            precision: "fp32" (fp32 FMA everywhere), "bf16" (bf16 q/k/v + KV caches,
                tensor-core context contraction, fp32 elsewhere) or None: follow the
                dtype handed to ``init_kv_cache`` / the inputs.
        """
        self.embedder = embedder
        self.backbone = backbone
        self.head = head
        self.ar_tokens = ar_tokens
        if backend not in ("flex_attention", "triton_shared_context"):
            raise ValueError(f"Unsupported backend: {backend}")
        if precision not in (None, "fp32", "bf16"):
            raise ValueError(f"Unsupported precision: {precision}")
        self.backend = backend
        self.precision = precision

        self.seq_len = 0
        self.context_len = 0
        self.buffer_len = 0
        self.max_buffer_len = 0
        self._device = None
        self._dtype = None
        self._batch = 0
        self._max_seq = 0
        self._state: Optional[_lib.State] = None
        self._bufs = {}
        self.last_logdens: Optional[Tensor] = None
        self.last_components: Optional[Tensor] = None
        self.last_h2d_bytes = 0
        self._status_host: Optional[Tensor] = None
        self._status_event = None

    @classmethod
    def from_trained_model(cls, model, backend: str = "flex_attention",
                           precision: Optional[str] = None) -> "ARTabPFNPredictor":
        return cls(model.embedder, model.backbone, model.head, model.ar_tokens, backend=backend,
                   precision=precision)

    # ------------------------------------------------------------------ state
    @property
    def shared(self) -> bool:
        return self.backend == "triton_shared_context"

    def _packed(self, device):
        return packed_for(self, self.embedder, self.backbone, self.head, self.ar_tokens, device)

    def _cache_dtype(self, dtype: Optional[torch.dtype]) -> torch.dtype:
        if self.precision == "fp32":
            return torch.float32
        if self.precision == "bf16":
            return torch.bfloat16
        if dtype in (torch.bfloat16, torch.float16):
            return torch.bfloat16
        return torch.float32

    def _model_device(self) -> torch.device:
        d = next(self.backbone.parameters()).device
        return torch.device("cuda", torch.cuda.current_device()) if d.type == "cuda" and d.index is None else d

    def _work_device(self, t: Tensor) -> torch.device:
        """Inputs may live in host memory (pinned for asynchronous copies): the work then runs on
        the model's device and only what the path reads is copied."""
        return t.device if t.is_cuda else self._model_device()

    def _dev32(self, t: Tensor, device) -> Tensor:
        """fp32 contiguous copy of ``t`` on ``device``; host tensors are copied on the current
        stream and counted in ``last_h2d_bytes``."""
        t = t.detach()
        if not t.is_cuda:
            self.last_h2d_bytes += t.numel() * t.element_size()
            t = t.to(device, non_blocking=True)
        return t.to(torch.float32).contiguous()

    def init_kv_cache(self, batch_size: int, max_seq_len: int, device: Optional[torch.device] = None,
                      dtype: Optional[torch.dtype] = None) -> None:
        """Record the cache geometry.  ``max_seq_len`` is the buffer capacity for the
        shared backend and context + buffer capacity for the per-batch backend, as
        in the reference (inference.py:82-135).  Device memory is laid out once the
        context length is known (``prefill_context``) and then never re-allocated."""
        if device is None or dtype is None:
            param = next(self.backbone.parameters())
            device = device or param.device
            dtype = dtype or param.dtype
        self._device = torch.device(device)
        if self._device.type == "cuda" and self._device.index is None:
            self._device = torch.device("cuda", torch.cuda.current_device())
        self._dtype = dtype
        self._batch = int(batch_size)
        self._max_seq = int(max_seq_len)
        self.max_buffer_len = int(max_seq_len) if self.shared else 0
        self.seq_len = 0
        self.context_len = 0
        self.buffer_len = 0
        self._state = None

    def clear_cache(self) -> None:
        """Reset cache state (keeps allocated memory)."""
        self.seq_len = 0
        self.context_len = 0
        self.buffer_len = 0
        if self._state is not None:
            self._state.buffer_len = 0

    def _alloc(self, name: str, shape, dtype) -> Tensor:
        t = self._bufs.get(name)
        n = 1
        for s in shape:
            n *= int(s)
        if t is None or t.dtype != dtype or t.device != self._device or t.numel() < n:
            t = torch.zeros(max(n, 1), dtype=dtype, device=self._device)
            self._bufs[name] = t
        return t[:n].view(*shape)

    def _ensure_rows(self, rows: int) -> None:
        """Row workspaces (residual stream, queries, attention output, partials)."""
        st, pm = self._state, self._packed(self._device)
        if rows <= st.max_rows:
            return
        D, H, Dh = pm.d_model, pm.n_heads, pm.head_dim
        rows = (rows + 127) // 128 * 128   # whole 128-row tiles: the tensor-core chain reads padded tiles
        cdt = torch.bfloat16 if st.dtype == _lib.BF16 else torch.float32
        st.x = self._alloc("x", (rows, D), torch.float32).data_ptr()
        st.x1 = self._alloc("x1", (rows, D), torch.float32).data_ptr()
        st.attn = self._alloc("attn", (rows, D), torch.float32).data_ptr()
        st.q = self._alloc("q", (rows, D), cdt).data_ptr()
        st.o_part = self._alloc("o_part", (_lib.MAX_SPLITS, rows, D), torch.float32).data_ptr()
        st.lse_part = self._alloc("lse_part", (_lib.MAX_SPLITS, rows, H), torch.float32).data_ptr()
        st.max_rows = rows
        st.max_splits = _lib.MAX_SPLITS

    def _layout(self, n_ctx: int) -> None:
        """Allocate the layout-fixed caches: context K [L,G,H,Ncp,Dh], context V
        (in bf16 transposed and split hi | lo: [L,G,H,2Dh,Ncp]; the exposed
        ``v_ctx_cache`` view is the hi part) and the private buffers [L,B,H,T,2,Dh]."""
        pm = self._packed(self._device)
        cdt = self._cache_dtype(self._dtype)
        B = self._batch
        G = 1 if self.shared else B
        T = self._max_seq if self.shared else max(self._max_seq - n_ctx, 0)
        L, H, Dh = pm.n_layers, pm.n_heads, pm.head_dim
        Ncp = _pad8(n_ctx)
        st = _lib.State()
        st.dtype = _lib.dtype_code(cdt)
        st.n_streams, st.n_groups, st.n_ctx, st.n_ctx_pad, st.max_buf = B, G, n_ctx, Ncp, T
        st.buffer_len, st.max_rows, st.max_splits = 0, 0, _lib.MAX_SPLITS
        k_ctx = self._alloc("k_ctx", (L, G, H, Ncp, Dh), cdt)
        if cdt == torch.bfloat16:
            v_ctx = self._alloc("v_ctx", (L, G, H, 2 * Dh, Ncp), cdt)  # hi | lo parts
        else:
            v_ctx = self._alloc("v_ctx", (L, G, H, Ncp, Dh), cdt)
        k_ctx.zero_()
        v_ctx.zero_()
        kv = self._alloc("kv_buf", (L, B, H, T, 2, Dh), cdt)
        st.k_ctx, st.v_ctx = k_ctx.data_ptr(), v_ctx.data_ptr()
        st.kv_buf = kv.data_ptr() if T > 0 else None
        st.status = self._alloc("status", (1,), torch.int32).data_ptr()
        self._state = st
        self.max_buffer_len = T
        # reference-shaped views on the layer modules (inference.py:113-118)
        for l, layer in enumerate(self.backbone.layers):
            kc = k_ctx[l, :, :, :n_ctx]
            vc = (v_ctx[l, :, :, :Dh].transpose(-1, -2)[:, :, :n_ctx] if cdt == torch.bfloat16
                  else v_ctx[l, :, :, :n_ctx])
            layer.k_ctx_cache = kc[0] if self.shared else kc
            layer.v_ctx_cache = vc[0] if self.shared else vc
            layer.k_buf_cache = kv[l, :, :, :, 0]
            layer.v_buf_cache = kv[l, :, :, :, 1]

    # ---------------------------------------------------------------- status
    def _mirror_status(self) -> None:
        """Queue a copy of the device status word (non-zero: a bounded device-side wait gave up and
        the results of that call are void) into pinned host memory behind the work just enqueued."""
        st = self._bufs.get("status")
        if st is None:
            return
        if self._status_host is None:
            self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._status_host.copy_(st, non_blocking=True)
        self._status_event = torch.cuda.current_stream(st.device).record_event()

    def last_status(self, wait: bool = True) -> int:
        """Status word of the most recent whole-path call: 0, or the code of the kernel whose wait ran
        out.  ``wait=False`` returns -1 while that call is still running instead of blocking."""
        if self._status_event is None:
            return 0
        if not wait and not self._status_event.query():
            return -1
        self._status_event.synchronize()
        return int(self._status_host.item())

    def _raise_if_timed_out(self) -> None:
        """Called at the start of every whole-path call: if the previous call has finished and one of
        its waits ran out, raise (ARTAB_ETIMEOUT) instead of silently continuing; never blocks."""
        if self.last_status(wait=False) > 0:
            code = int(self._status_host.item())
            self._status_event = None
            st = self._bufs.get("status")
            if st is not None:
                st.zero_()
            raise _lib.ArtabError(f"artab error {_lib.ETIMEOUT}: a bounded device-side wait gave up in the previous "
                                  f"call (status {code}); its results are void")

    # --------------------------------------------------------------- prefill
    @torch.no_grad()
    def prefill_context(self, x_context: Tensor, y_context: Tensor) -> None:
        """Encode the context rows and fill the context K/V of every layer.
        x_context [B,Nc,F], y_context [B,Nc]."""
        lib = _lib.lib()
        if self._device is None:
            raise RuntimeError("init_kv_cache must be called before prefill_context")
        if x_context.is_cuda and x_context.device != self._device:
            raise ValueError("inputs must live on the cache device (or in host memory)")
        if self.shared:
            # only batch element 0 is the shared context (inference.py:191-193): a host tensor is
            # sliced before it is copied
            x_context, y_context = x_context[0:1], y_context[0:1]
        elif x_context.shape[0] != self._batch:
            raise ValueError("batch size differs from init_kv_cache")
        G, Nc, F = x_context.shape
        self._layout(Nc)
        self._ensure_rows(max(G * Nc, 2 * self._batch))
        xc = self._dev32(x_context, self._device)
        yc = self._dev32(y_context, self._device).reshape(G, Nc)
        pm = self._packed(self._device)
        _lib.check(lib.artab_prefill(pm.ref, C.byref(self._state), _lib.ptr(xc), _lib.ptr(yc), F,
                                     _lib.stream_ptr()))
        self.context_len = Nc
        self.buffer_len = 0
        self.seq_len = Nc
        self._prefill_batch_size = self._batch

    def prefill_context_shared(self, x_context: Tensor, y_context: Tensor) -> None:
        self.prefill_context(x_context, y_context)

    # ---------------------------------------------------------------- decode
    @torch.no_grad()
    def transformer_decode(self, embedding: Tensor, commit: int) -> Tensor:
        """embedding [B,N,D] (N = 1: target; N = 2: buffer, target) -> [B,N,D] after
        the final norm; ``commit`` buffer rows are kept in the private cache."""
        lib = _lib.lib()
        B, N, D = embedding.shape
        if N not in (1, 2):
            raise ValueError("Shared-context decode only supports N=1 (target) or N=2 (buffer, target).")
        if self._state is None:
            raise RuntimeError("prefill_context must be called before decoding")
        if self.buffer_len + commit > self.max_buffer_len:
            raise ValueError("Shared-context buffer cache exceeded; increase max buffer length.")
        self._ensure_rows(B * N)
        x = embedding.detach().to(torch.float32).contiguous()
        z = torch.empty(B, N, D, device=embedding.device, dtype=torch.float32)
        pm = self._packed(self._device)
        self._state.buffer_len = self.buffer_len
        _lib.check(lib.artab_decode_embedded(pm.ref, C.byref(self._state), _lib.ptr(x), N, commit, _lib.ptr(z),
                                             _lib.stream_ptr()))
        self.buffer_len = int(self._state.buffer_len)
        self.seq_len = self.context_len + self.buffer_len
        return z.to(embedding.dtype)

    @torch.no_grad()
    def autoregressive_decode(self, x_target: Tensor, prev_x: Optional[Tensor] = None,
                              prev_y: Optional[Tensor] = None, ar_idx: int = 0) -> Tensor:
        """Decode one target, optionally with the previous prediction as buffer
        element; returns the sampled y [B,1] (inference.py:279-320)."""
        target_emb = self.embedder.embed_target(x_target)
        if prev_x is not None and prev_y is not None:
            buffer_emb = self.embedder.embed_buffer(prev_x, prev_y)
            buffer_emb = buffer_emb + self.ar_tokens[ar_idx].to(buffer_emb.dtype)
            embedding = torch.cat([buffer_emb, target_emb], dim=1)
            commit = 1
        else:
            embedding = target_emb
            commit = 0
        z = self.transformer_decode(embedding, commit=commit)
        y_pred = self.head.sample(z[:, -1:, :])
        return y_pred[:, :, 0, 0]

    def draw_variates(self, n_steps: int, batch: int, device, dtype=torch.float32) -> Tuple[Tensor, Tensor]:
        """Pre-draw the random numbers of a whole sampling run from torch's current
        generator in exactly the order the reference consumes them: per step one
        Exp(1) fill of [B,K] (inside torch.multinomial) and then one N(0,1) fill of
        [B,1,1,1] (model.py:257, 265).  The draws do not depend on model outputs."""
        K = int(self.head.num_components)
        expo = torch.empty(n_steps, batch, K, device=device, dtype=dtype)
        normal = torch.empty(n_steps, batch, device=device, dtype=dtype)
        for t in range(n_steps):
            expo[t].exponential_(1)
            normal[t].normal_()   # the same fill as torch.randn(batch, 1, 1, 1): same element count, same stream
        return expo, normal

    @torch.no_grad()
    def sample_sequence(self, x_context: Tensor, y_context: Tensor, x_target: Tensor,
                        variates: Optional[Tuple[Tensor, Tensor]] = None) -> Tensor:
        """Predict all targets autoregressively: x_context [B,Nc,F], y_context [B,Nc],
        x_target [B,Nt,F] -> y_pred [B,Nt].

        ``variates = (expo [Nt,B,K], normal [Nt,B])`` replays given random numbers;
        by default they are drawn from torch's generator in the reference's order.
        The log density of each drawn value and the chosen component are kept in
        ``last_logdens`` / ``last_components`` ([B,Nt]).

        The inputs may also be host tensors (pinned memory makes the copies asynchronous):
        the work runs on the model's device, the result stays there, and only what the path
        reads is copied - with the shared-context backend that is batch element 0 of the
        context, not B copies of it (``last_h2d_bytes`` counts the bytes)."""
        lib = _lib.lib()
        self._raise_if_timed_out()
        B, Nc, F = x_context.shape
        Nt = x_target.shape[1]
        device, dtype = self._work_device(x_context), x_context.dtype
        self.last_h2d_bytes = 0
        if self.shared:
            self.init_kv_cache(B, Nt, device, dtype)
        else:
            self.init_kv_cache(B, Nc + Nt, device, dtype)
        drawn = None
        if variates is None:
            # The draws depend on nothing the model computes, so their launches (two small fills per
            # step) go to a side stream AFTER the prefill has been queued: the device runs the
            # prefill while the host is still issuing fills.  Torch advances its generator when a
            # fill is launched and the prefill draws nothing, so the values are those of the same
            # fills issued anywhere else in this call.
            main = torch.cuda.current_stream(device)
            side = self._bufs.get("side_stream")
            if side is None or side.device != device:
                side = self._bufs["side_stream"] = torch.cuda.Stream(device=device)
            K = int(self.head.num_components)
            expo = torch.empty(Nt, B, K, device=device, dtype=torch.float32)     # owned by the main stream
            normal = torch.empty(Nt, B, device=device, dtype=torch.float32)
            fresh = main.record_event()      # whatever used this memory before has finished by here
        self.prefill_context(x_context, y_context)
        if variates is None:
            side.wait_event(fresh)
            drawn = {}

            def issue_draws(t0):
                """Fills of steps [t0, t0 + 16) on the side stream; decode step t0 waits for them."""
                if t0 >= Nt or t0 in drawn:
                    return
                with torch.cuda.stream(side):
                    for t in range(t0, min(t0 + 16, Nt)):
                        expo[t].exponential_(1)
                        normal[t].normal_()
                    drawn[t0] = side.record_event()

            issue_draws(0)
            variates = (expo, normal)
        expo = variates[0].detach().to(device=device, dtype=torch.float32).contiguous()
        normal = variates[1].detach().to(device=device, dtype=torch.float32).contiguous()
        K = int(self.head.num_components)
        if expo.shape != (Nt, B, K) or normal.shape != (Nt, B):
            raise ValueError("variates must be (expo [Nt,B,K], normal [Nt,B])")
        xt = self._dev32(x_target, device)
        samples = torch.zeros(B, Nt, device=device, dtype=torch.float32)
        logdens = torch.zeros(B, Nt, device=device, dtype=torch.float32)
        comp = torch.zeros(B, Nt, device=device, dtype=torch.int32)
        pm = self._packed(device)
        st = self._state
        stream = _lib.stream_ptr()
        for t in range(Nt):
            if drawn is not None and t % 16 == 0:
                issue_draws(t + 16)      # the host stays one chunk ahead of the decode steps it launches
                torch.cuda.current_stream(device).wait_event(drawn[t])
            _lib.check(lib.artab_decode_step(pm.ref, C.byref(st), _lib.ptr(xt), F, Nt, t, _lib.ptr(samples),
                                             _lib.ptr(expo[t]), _lib.ptr(normal[t]), _lib.ptr(logdens),
                                             _lib.ptr(comp), stream))
        self.buffer_len = int(st.buffer_len)
        self.seq_len = self.context_len + self.buffer_len
        self.last_logdens = logdens
        self.last_components = comp
        self._mirror_status()
        return samples.to(dtype)

    # ------------------------------------------------------- teacher forcing
    @torch.no_grad()
    def evaluate_joint_density(self, x_context: Tensor, y_context: Tensor, x_target: Tensor,
                               y_target: Tensor) -> Tensor:
        """Teacher-forced log density of every target, [B,Nt], in one block-causal pass."""
        lib = _lib.lib()
        self._raise_if_timed_out()
        B, Nc, F = x_context.shape
        Nt = x_target.shape[1]
        device, dtype = self._work_device(x_context), x_context.dtype
        self.last_h2d_bytes = 0
        if self.shared:
            self.init_kv_cache(B, Nt, device, dtype)
        else:
            # the reference reserves Nc + 2*Nt; only the Nt buffer rows are ever cached
            self.init_kv_cache(B, Nc + Nt, device, dtype)
        self.prefill_context(x_context, y_context)
        self._ensure_rows(2 * B * Nt)
        xt = self._dev32(x_target, device)
        yt = self._dev32(y_target, device).reshape(B, Nt)
        out = torch.empty(B, Nt, device=device, dtype=torch.float32)
        pm = self._packed(device)
        _lib.check(lib.artab_teacher_forcing(pm.ref, C.byref(self._state), _lib.ptr(xt), _lib.ptr(yt), F, Nt,
                                             _lib.ptr(out), _lib.stream_ptr()))
        self.buffer_len = int(self._state.buffer_len)
        self.seq_len = self.context_len + self.buffer_len
        self._mirror_status()
        return out.to(dtype)

    # -------------------------------------------------------- masked forward
    @torch.no_grad()
    def forward_masked(self, x_context: Tensor, y_context: Tensor, x_buffer: Tensor, y_buffer: Tensor,
                       x_target: Tensor, y_target: Tensor, visible) -> Tensor:
        """Per-target log density [B,Nt] of the reference's training forward
        (model.py:317-369) for inference: context rows see the context; token j of
        [Buffer_0..Buffer_{Nb-1}, Target_0..Target_{Nt-1}] sees the context plus the first
        ``visible[j]`` buffer rows (``RowMask.visible`` of ``create_row_mask``)."""
        lib = _lib.lib()
        self._raise_if_timed_out()
        B, Nc, F = x_context.shape
        Nb, Nt = x_buffer.shape[1], x_target.shape[1]
        if len(visible) != Nb + Nt:
            raise ValueError(f"visible must list {Nb + Nt} counts (buffer rows, then target rows)")
        if Nb > self.ar_tokens.shape[0]:
            raise ValueError(f"{Nb} buffer rows but only {self.ar_tokens.shape[0]} AR position tokens")
        device, dtype = self._work_device(x_context), x_context.dtype
        self.last_h2d_bytes = 0
        if self.shared:
            self.init_kv_cache(B, Nb, device, dtype)
        else:
            self.init_kv_cache(B, Nc + Nb, device, dtype)
        self.prefill_context(x_context, y_context)
        self._ensure_rows(B * (Nb + Nt))
        f32 = lambda t, *shape: self._dev32(t, device).reshape(*shape)
        xb, yb = f32(x_buffer, B, Nb, F), f32(y_buffer, B, Nb)
        xt, yt = f32(x_target, B, Nt, F), f32(y_target, B, Nt)
        vis = torch.tensor([int(v) for v in visible], dtype=torch.int32, device=device)
        out = torch.empty(B, Nt, device=device, dtype=torch.float32)
        pm = self._packed(device)
        _lib.check(lib.artab_forward_masked(pm.ref, C.byref(self._state), _lib.ptr(xb), _lib.ptr(yb), _lib.ptr(xt),
                                            _lib.ptr(yt), F, Nb, Nt, _lib.ptr(vis), _lib.ptr(out),
                                            _lib.stream_ptr()))
        self.buffer_len = int(self._state.buffer_len)
        self.seq_len = self.context_len + self.buffer_len
        self._mirror_status()
        return out.to(dtype)
