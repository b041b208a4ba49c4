"""HybridCache: the device-side DualCache (paged F16 KV + FP32 DeltaNet state +
conv windows) and the decode step over layer_types[], through rl_cache_* /
rl_stack_* of the C ABI.  Mirrors rapidllm::DualCache
(include/rapidllm/runtime/dual_cache.h:11-39) and the scheduler loop of
Session::forward_hidden (src/runtime/session.cpp:325-411).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import CacheConfig, StackIO, check, lib

QWEN35_LAYER_TYPES = [_lib.RL_LAYER_LINEAR_ATTENTION] * 3 + [_lib.RL_LAYER_FULL_ATTENTION]


class _DevView:
    """Zero-copy torch view of library-owned device memory."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr,
                                         "data": (int(ptr), False), "version": 2}


def _view(ptr, shape, dtype):
    typestr = {torch.float32: "<f4", torch.float16: "<f2", torch.int32: "<i4", torch.uint8: "|u1"}[dtype]
    return torch.as_tensor(_DevView(ptr, shape, typestr), device="cuda")


class HybridCache:
    def __init__(self, layer_types, n_pages, n_slots, max_batch, max_pages_per_seq,
                 max_seq_len=None, n_q=24, n_kv=4, head_dim=256, n_v=48, n_k=16, dk=128, dv=128,
                 conv_k=4, head_map=_lib.RL_HEADS_GROUPED, kv_dtype=_lib.RL_KV_F16, wht_len=128, window_tokens=0,
                 tq_signs=None):
        self.layer_types = list(layer_types)
        self.n_attn = sum(1 for t in self.layer_types if t == _lib.RL_LAYER_FULL_ATTENTION)
        self.n_delta = len(self.layer_types) - self.n_attn
        self.n_q, self.n_kv, self.head_dim = n_q, n_kv, head_dim
        self.n_v, self.n_k, self.dk, self.dv, self.conv_k = n_v, n_k, dk, dv, conv_k
        self.conv_dim = 2 * n_k * dk + n_v * dv
        self.n_pages, self.n_slots, self.max_batch = n_pages, n_slots, max_batch
        self.max_pages_per_seq = max_pages_per_seq
        self.max_seq_len = max_seq_len or max_pages_per_seq * 64
        self.kv_dtype, self.wht_len, self.window_tokens = kv_dtype, wht_len, window_tokens
        self.window_pages = -(-window_tokens // 64) if kv_dtype == _lib.RL_KV_Q8K_TQ3V else 0
        arr = (C.c_int * len(self.layer_types))(*self.layer_types)
        signs = None if tq_signs is None else tq_signs.detach().cpu().float().contiguous()   # HOST [256]
        cfg = CacheConfig(n_layers=len(self.layer_types), layer_types=arr, n_q=n_q, n_kv=n_kv,
                          head_dim=head_dim, kv_dtype=kv_dtype, wht_len=wht_len, window_tokens=window_tokens,
                          tq_signs=None if signs is None else signs.data_ptr(), page_tokens=64,
                          n_pages=n_pages, n_v=n_v, n_k=n_k, dk=dk, dv=dv, conv_k=conv_k,
                          head_map=head_map, n_slots=n_slots, max_batch=max_batch,
                          max_pages_per_seq=max_pages_per_seq, max_seq_len=self.max_seq_len)
        h = C.c_void_p()
        check(lib().rl_cache_create(C.byref(cfg), C.byref(h)))
        self._h = h

    def close(self):
        if getattr(self, "_h", None):
            lib().rl_cache_destroy(self._h)
            self._h = None

    __del__ = close

    @property
    def bytes(self):
        return lib().rl_cache_bytes(self._h)

    def k_pool(self, i):
        if self.kv_dtype == _lib.RL_KV_Q8K_TQ3V:           # record pool of the compact cache (bytes)
            return _view(lib().rl_cache_k_pool(self._h, i), (self.n_pages, self.n_kv, lib().rl_kv_compact_page_bytes()),
                         torch.uint8)
        return _view(lib().rl_cache_k_pool(self._h, i), (self.n_pages, self.n_kv, 64 * 256), torch.float16)

    def window_pools(self, i):
        """(K, V) F16 window pools of attention layer i beside a compact cache: slot s owns pages
        [s * window_pages, (s + 1) * window_pages)."""
        shape = (self.n_slots * self.window_pages, self.n_kv, 64 * 256)
        return (_view(lib().rl_cache_window_k_pool(self._h, i), shape, torch.float16),
                _view(lib().rl_cache_window_v_pool(self._h, i), shape, torch.float16))

    def v_pool(self, i):
        return _view(lib().rl_cache_v_pool(self._h, i), (self.n_pages, self.n_kv, 64 * 256), torch.float16)

    def state(self, i):
        return _view(lib().rl_cache_state(self._h, i), (self.n_slots, self.n_v, self.dk, self.dv), torch.float32)

    def conv(self, i):
        return _view(lib().rl_cache_conv(self._h, i), (self.n_slots, self.conv_dim, self.conv_k), torch.float32)

    def conv_windows(self, i):
        """The conv windows of DeltaNet layer i in the reference's form [n_slots][conv_dim][4], oldest
        tap first (a copy: the cache keeps them as rings, see rl_gdn_decode)."""
        out = torch.empty(self.n_slots, self.conv_dim, self.conv_k, dtype=torch.float32, device="cuda")
        check(lib().rl_cache_conv_export(self._h, i, C.c_void_p(out.data_ptr()),
                                         C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return out

    def set_conv_windows(self, i, windows):
        """Load layer i's windows from the reference's form [n_slots][conv_dim][4]."""
        w = windows.to(device="cuda", dtype=torch.float32).contiguous()
        assert tuple(w.shape) == (self.n_slots, self.conv_dim, self.conv_k)
        check(lib().rl_cache_conv_import(self._h, i, C.c_void_p(w.data_ptr()),
                                         C.c_void_p(torch.cuda.current_stream().cuda_stream)))

    def zero(self):
        check(lib().rl_cache_zero(self._h, C.c_void_p(torch.cuda.current_stream().cuda_stream)))

    @property
    def launches_per_step(self):
        return lib().rl_stack_launches_per_step(self._h)

    def set_graph(self, enable: bool):
        """Graph replay of decode() (on by default; off while timing is on)."""
        check(lib().rl_stack_set_graph(self._h, int(enable)))

    def set_timing(self, enable: bool):
        check(lib().rl_stack_set_timing(self._h, int(enable)))

    def timing(self):
        """ms of the last step per kernel family, summed over the layers."""
        ms = (C.c_float * 5)()
        check(lib().rl_stack_timing(self._h, ms))
        return dict(zip(("kv_append", "attn_decode", "attn_combine", "conv1d_update", "delta_rule"),
                        list(ms)))

    def io_shapes(self, batch):
        """Tensor name -> shape of one decode step's inputs and outputs."""
        A, D, B = self.n_attn, self.n_delta, batch
        return {"attn_q": (A, B, self.n_q, 256), "attn_gate": (A, B, self.n_q, 256),
                "attn_k": (A, B, self.n_kv, 256), "attn_v": (A, B, self.n_kv, 256),
                "attn_o": (A, B, self.n_q, 256), "delta_qkv": (D, B, self.conv_dim),
                "delta_beta": (D, B, self.n_v), "delta_g": (D, B, self.n_v),
                "delta_o": (D, B, self.n_v, self.dv), "conv_w": (D, self.conv_dim, self.conv_k),
                "page_table": (B, self.max_pages_per_seq), "pos": (B,), "slot_ids": (B,),
                "attn_ml": (A, B, self.n_q, 2)}

    def _io(self, t, batch, cuda):
        io = StackIO(batch=batch)
        io.no_append = int(bool(t.get("no_append", False)))
        io.kv_window_ok = int(bool(t.get("kv_window_ok", False)))
        glue = t.get("glue")
        if glue is not None:
            # raw projections and small weights: the element-wise steps run inside the step (rl_stack_glue)
            g = _lib.StackGlue(rotary_dim=int(glue.get("rotary_dim", 64)), theta=float(glue.get("theta", 1e7)),
                               rms_eps=float(glue.get("rms_eps", 1e-6)))
            for name in ("attn_qg", "attn_k_raw", "q_norm", "k_norm", "delta_a", "delta_b", "A_log", "dt_bias",
                         "delta_z", "gnorm"):
                x = glue.get(name)
                if x is None:
                    continue
                if not (x.is_cuda and x.is_contiguous() and x.dtype == torch.float32):
                    raise _lib.RlError(6, f"glue.{name}: need a contiguous fp32 CUDA tensor")
                setattr(g, name, x.data_ptr())
            io.glue = C.addressof(g)
            io._glue_keepalive = g
        for name in ("attn_q", "attn_gate", "attn_k", "attn_v", "attn_o", "delta_qkv", "delta_beta",
                     "delta_g", "delta_o", "conv_w", "page_table", "pos", "slot_ids", "attn_ml"):
            x = t.get(name)
            if x is None:
                continue
            if x.is_cuda != cuda or not x.is_contiguous():
                raise _lib.RlError(6, f"{name}: need a contiguous {'CUDA' if cuda else 'host'} tensor")
            want = torch.int32 if name in ("page_table", "pos", "slot_ids") else torch.float32
            if x.dtype != want:
                raise _lib.RlError(6, f"{name}: need dtype {want}")
            setattr(io, name, x.data_ptr())
        return io

    def decode(self, tensors: dict, batch: int):
        """One step over layer_types[] with device tensors (rl_stack_decode)."""
        io = self._io(tensors, batch, True)
        check(lib().rl_stack_decode(self._h, C.byref(io), C.c_void_p(torch.cuda.current_stream().cuda_stream)))

    def prefill_shapes(self, T):
        """Tensor name -> (shape, dtype) of one prefill chunk's inputs and outputs."""
        A, D = self.n_attn, self.n_delta
        bf, f32 = torch.bfloat16, torch.float32
        return {"attn_q": ((A, T, self.n_q, 256), bf), "attn_k": ((A, T, self.n_kv, 256), bf),
                "attn_v": ((A, T, self.n_kv, 256), bf), "attn_gate": ((A, T, self.n_q, 256), f32),
                "attn_o": ((A, T, self.n_q, 256), f32), "delta_qkv": ((D, T, self.conv_dim), f32),
                "delta_beta": ((D, T, self.n_v), f32), "delta_g": ((D, T, self.n_v), f32),
                "delta_o": ((D, T, self.n_v, self.dv), f32), "conv_w": ((D, self.conv_dim, self.conv_k), f32)}

    def prefill(self, tensors: dict, page_table_row, slot: int, pos0: int, T: int, workspace=None):
        """One chunk of one sequence's prompt through every layer (rl_stack_prefill): device tensors
        shaped as prefill_shapes(T); page_table_row int32 [max_pages_per_seq] on the device."""
        io = _lib.StackPrefillIO(slot=slot, pos0=pos0, T=T)
        shapes = self.prefill_shapes(T)
        for name, (shape, dtype) in shapes.items():
            x = tensors.get(name)
            if x is None:
                continue
            if not (x.is_cuda and x.is_contiguous() and x.dtype == dtype and tuple(x.shape) == shape):
                raise _lib.RlError(6, f"{name}: need a contiguous CUDA tensor {shape} of {dtype}")
            setattr(io, name, x.data_ptr())
        if not (page_table_row.is_cuda and page_table_row.dtype == torch.int32 and page_table_row.is_contiguous()
                and page_table_row.numel() == self.max_pages_per_seq):
            raise _lib.RlError(6, "page_table_row: need int32 [max_pages_per_seq] on the device")
        io.page_table_row = page_table_row.data_ptr()
        need = lib().rl_stack_prefill_workspace_bytes(self._h, pos0, T)
        if workspace is None or workspace.numel() < need:
            workspace = torch.empty(max(need, 256), dtype=torch.uint8, device=page_table_row.device)
        check(lib().rl_stack_prefill(self._h, C.byref(io), C.c_void_p(workspace.data_ptr()), workspace.numel(),
                                     C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return workspace

    def gather_shapes(self, batch, n_ranks):
        """Tensor name -> shape of the buffers a sharded step gathers into (rl_stack_gather)."""
        A, D, B, W = self.n_attn, self.n_delta, batch, n_ranks
        return {"attn_o_all": (A, W, B, self.n_q, 256), "delta_o_all": (D, W, B, self.n_v, self.dv),
                "attn_ml_all": (A, W, B, self.n_q, 2), "attn_o_final": (A, B, self.n_q, 256)}

    def set_gather(self, comm, tensors: dict | None, layers_per_exchange: int = 0, reserve_sms: int = 0):
        """Attach the all-gather of the step's outputs over `comm` (a Comm) to decode() /
        decode_host(); tensors: device buffers shaped as gather_shapes().  None detaches."""
        if comm is None or tensors is None:
            check(lib().rl_stack_set_gather(self._h, None))
            self._gather = None
            return
        g = _lib.StackGather(comm=comm.handle, layers_per_exchange=layers_per_exchange, reserve_sms=reserve_sms)
        for name in ("attn_o_all", "delta_o_all", "attn_ml_all", "attn_o_final"):
            x = tensors.get(name)
            if x is None:
                continue
            if not (x.is_cuda and x.is_contiguous() and x.dtype == torch.float32):
                raise _lib.RlError(6, f"{name}: need a contiguous fp32 CUDA tensor")
            setattr(g, name, x.data_ptr())
        check(lib().rl_stack_set_gather(self._h, C.byref(g)))
        self._gather = (comm, tensors)           # keep the buffers alive

    def set_conv_w(self, host_w: torch.Tensor):
        check(lib().rl_stack_set_conv_w(self._h, C.c_void_p(host_w.data_ptr())))

    def decode_host(self, tensors: dict, batch: int):
        """One step with HOST tensors (pinned for speed): H2D, step, D2H (rl_stack_decode_host)."""
        io = self._io(tensors, batch, False)
        check(lib().rl_stack_decode_host(self._h, C.byref(io)))


class Comm:
    """rl_comm: the NCCL communicator of the ranks that share a step.  `exchange_id` is any
    callable that takes the 128-byte id made on rank 0 (bytes, or None on other ranks) and returns
    it on every rank, e.g. a torch.distributed broadcast."""

    def __init__(self, rank: int, n_ranks: int, exchange_id):
        buf = (C.c_ubyte * _lib.COMM_ID_BYTES)()
        if rank == 0:
            check(lib().rl_comm_unique_id(buf))
        raw = exchange_id(bytes(buf) if rank == 0 else None)
        buf = (C.c_ubyte * _lib.COMM_ID_BYTES).from_buffer_copy(raw)
        h = C.c_void_p()
        check(lib().rl_comm_create(buf, rank, n_ranks, C.byref(h)))
        self.handle, self.rank, self.n_ranks = h, rank, n_ranks

    def close(self):
        if getattr(self, "handle", None):
            lib().rl_comm_destroy(self.handle)
            self.handle = None
