"""Host-side mirror of the C ABI: the MoE layer handle and the stage entry points on torch tensors.

torch is used for device memory, streams and (by callers) torch.distributed; every computation goes through
libaristos_moe.so. Nothing here falls back to PyTorch ops."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from .config import AristosConfig

_TORCH_DTYPE = {_lib.DTYPE_F32: torch.float32, _lib.DTYPE_TF32: torch.float32, _lib.DTYPE_BF16: torch.bfloat16,
                _lib.DTYPE_F16: torch.float16, _lib.DTYPE_FP8_E4M3: torch.bfloat16}   # fp8: activations are bf16
# storage type -> dtype code; fp32 tensors mean exact fp32 math unless a call asks for tf32 explicitly
_ARISTOS_DTYPE = {torch.float32: _lib.DTYPE_F32, torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_F16}


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return None
    if not t.is_contiguous():
        raise ValueError("tensors passed to the C ABI must be contiguous")
    return C.c_void_p(t.data_ptr())


def _stream_ptr(stream: Optional[torch.cuda.Stream] = None):
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


def _dt(t: torch.Tensor) -> int:
    try:
        return _ARISTOS_DTYPE[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported tensor dtype {t.dtype}") from None


def nccl_unique_id() -> bytes:
    buf = C.create_string_buffer(128)
    _lib.check(_lib.load().aristos_nccl_unique_id(buf))
    return buf.raw


def fill_normal(t: torch.Tensor, mean: float, std: float, seed: int, stream_id: int) -> torch.Tensor:
    _lib.check(_lib.load().aristos_fill_normal(_ptr(t), t.numel(), mean, std, seed, stream_id, _dt(t), _stream_ptr()))
    return t


def zipf_prior(num_experts: int, s: float) -> torch.Tensor:
    """The per-expert gate prior of `gate_bias_zipf_s` (-s ln(e + 1), fp32, host) as the layer builds it itself."""
    b = (C.c_float * num_experts)()
    _lib.check(_lib.load().aristos_zipf_bias_host(b, num_experts, float(s)))
    return torch.tensor(list(b), dtype=torch.float32)


def interleaved_expert_prior(prior: torch.Tensor, world: int) -> torch.Tensor:
    """Round-robin expert placement for a per-expert gate prior given in the experts' own order (entry e = expert e).

    A rank owns a contiguous block of E / world expert slots (rank r: slots [r E/world, (r + 1) E/world)). Holding
    expert e in slot (e % world) * (E / world) + e // world gives consecutive experts to different ranks, so the hot
    experts of a skewed prior do not all land on rank 0. Returns the prior indexed by slot - the gate_bias argument
    of the forward; the gate and expert weights of slot p are then those of expert (p % (E/world)) * world +
    p // (E/world). With world = 1 the prior is returned unchanged."""
    E = prior.numel()
    if world <= 1:
        return prior.clone()
    if E % world != 0:
        raise ValueError("the number of experts must be a multiple of the number of ranks")
    El = E // world
    slots = torch.arange(E)
    expert_of_slot = (slots % El) * world + slots // El
    return prior[expert_of_slot].clone()


def synthetic_tensors(cfg: AristosConfig, rank: int = 0, world: int = 1):
    """Seeded synthetic inputs of one rank, generated on the device: x ~ N(0,1) (a different stream per rank),
    gate weights and this rank's expert weights ~ N(0, 0.02). Expert e draws from its own Philox streams, so the
    shards of every world size are slices of the same global weights. Returns (x, w_gate, w1, w3, w2, scales);
    for torch_dtype 4 the expert weights are e4m3 codes (uint8) and scales holds their 128x128-block scales
    [s1 | s3 | s2], otherwise scales is None."""
    fp8 = cfg.torch_dtype == _lib.DTYPE_FP8_E4M3
    dt = _TORCH_DTYPE[cfg.torch_dtype]
    S, H, I, E = cfg.S, cfg.hidden_size, cfg.intermediate_size, cfg.num_experts
    El = E // world
    swiglu = cfg.hidden_act == _lib.ACT_SWIGLU
    new = lambda *shape: torch.empty(shape, dtype=dt, device="cuda")
    x = fill_normal(new(S, H), 0.0, 1.0, cfg.seed, 0 if rank == 0 else 0x1000 + rank)
    wg = fill_normal(new(E, H), 0.0, 0.02, cfg.seed, 1)

    def expert_tensor(rows, cols, which):
        if not fp8:
            w = new(El, rows, cols)
            for el in range(El):
                fill_normal(w[el], 0.0, 0.02, cfg.seed, 16 * (rank * El + el + 1) + which)
            return w, None
        q = torch.empty((El, rows, cols), dtype=torch.uint8, device="cuda")
        sc = torch.empty((El, (rows + 127) // 128, cols // 128), dtype=torch.float32, device="cuda")
        tmp = new(rows, cols)
        for el in range(El):          # one expert at a time: the bf16 originals never exist all at once
            fill_normal(tmp, 0.0, 0.02, cfg.seed, 16 * (rank * El + el + 1) + which)
            qe, se = quantize_fp8(tmp, 128)
            q[el].copy_(qe)
            sc[el].copy_(se)
        return q, sc

    w1, s1 = expert_tensor(I, H, 2)
    w3, s3 = expert_tensor(I, H, 3) if swiglu else (None, None)
    w2, s2 = expert_tensor(H, I, 4)
    scales = torch.cat([t.reshape(-1) for t in (s1, s3, s2) if t is not None]).contiguous() if fp8 else None
    return x, wg, w1, w3, w2, scales


# ---- stage entry points ---------------------------------------------------------------------------------------------
def gate_topk(x, w_gate, k: int, gate_fn: int = 0, renorm: int = 0, gate_bias=None, want_logits: bool = False):
    S, H = x.shape
    E = w_gate.shape[0]
    idx = torch.empty((S, k), dtype=torch.int32, device=x.device)
    w = torch.empty((S, k), dtype=torch.float32, device=x.device)
    logits = torch.empty((S, E), dtype=torch.float32, device=x.device) if want_logits else None
    _lib.check(_lib.load().aristos_gate_topk(_ptr(x), _ptr(w_gate), _ptr(gate_bias), S, H, E, k, gate_fn, renorm,
                                             _dt(x), _ptr(idx), _ptr(w), _ptr(logits), _stream_ptr()))
    return (idx, w, logits) if want_logits else (idx, w)


def gate_topk_screened(x, w_gate, k: int, gate_fn: int = 0, renorm: int = 0, gate_bias=None):
    """aristos_gate_topk_screened: tensor-core screen + exact evaluation of the experts that can still reach the
    top k (the layer's gate for 16-bit inputs and 32 <= E <= 256). Returns (topk_idx, topk_w, status word)."""
    S, H = x.shape
    E = w_gate.shape[0]
    lib = _lib.load()
    idx = torch.empty((S, k), dtype=torch.int32, device=x.device)
    w = torch.empty((S, k), dtype=torch.float32, device=x.device)
    nbytes = lib.aristos_gate_scratch_bytes(S, E)
    scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=x.device)
    status = torch.zeros(1, dtype=torch.int32, device=x.device)
    _lib.check(lib.aristos_gate_topk_screened(_ptr(x), _ptr(w_gate), _ptr(gate_bias), S, H, E, k, gate_fn, renorm,
                                              _dt(x), _ptr(idx), _ptr(w), _ptr(scratch), nbytes, _ptr(status),
                                              _stream_ptr()))
    return idx, w, status


def dispatch(topk_idx, E: int, cap: int):
    S, k = topk_idx.shape
    dev = topk_idx.device
    lib = _lib.load()
    nbytes = lib.aristos_dispatch_scratch_bytes(S, k, E)
    scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
    count = torch.empty(E, dtype=torch.int32, device=dev)
    slot_of = torch.empty((S, k), dtype=torch.int32, device=dev)
    tos = torch.empty(E * cap, dtype=torch.int32, device=dev)
    _lib.check(lib.aristos_dispatch(_ptr(topk_idx), S, k, E, cap, _ptr(count), _ptr(slot_of), _ptr(tos),
                                    _ptr(scratch), nbytes, _stream_ptr()))
    return count, slot_of, tos


def dispatch_static(topk_idx, E: int, cap: int):
    """aristos_dispatch_static: the dispatch for callers that cannot allocate device memory (the library's built-in
    64 KiB scratch; S*k <= 131072, E <= 256). The outputs are still the caller's (here: torch) buffers."""
    S, k = topk_idx.shape
    dev = topk_idx.device
    count = torch.empty(E, dtype=torch.int32, device=dev)
    slot_of = torch.empty((S, k), dtype=torch.int32, device=dev)
    tos = torch.empty(E * cap, dtype=torch.int32, device=dev)
    _lib.check(_lib.load().aristos_dispatch_static(_ptr(topk_idx), S, k, E, cap, _ptr(count), _ptr(slot_of),
                                                   _ptr(tos), _stream_ptr()))
    return count, slot_of, tos


def permute(x, slot_of, nslots: int, zero: bool = False):
    S, H = x.shape
    k = slot_of.shape[1]
    xg = (torch.zeros if zero else torch.empty)((nslots, H), dtype=x.dtype, device=x.device)
    _lib.check(_lib.load().aristos_permute(_ptr(x), _ptr(slot_of), S, k, H, _dt(x), _ptr(xg), _stream_ptr()))
    return xg


def expert_ffn(xg, count, w1, w3, w2, hidden_act: int, *, experts: Optional[int] = None, row_begin: int = 0,
               row_end: Optional[int] = None, sm_limit: int = 0, dev_status=None, y=None, h=None, b1=None, b3=None,
               b2=None, dtype: Optional[int] = None):
    """xg (groups, rows, H); w1/w3 (experts, I, H); w2 (experts, H, I); optional biases b1/b3 (experts, I),
    b2 (experts, H) -> y (groups, rows, H)."""
    groups, rows, H = xg.shape
    I = w1.shape[1]
    experts = w1.shape[0] if experts is None else experts
    row_end = rows if row_end is None else row_end
    if h is None:
        h = torch.empty((groups, rows, I), dtype=xg.dtype, device=xg.device)
    if y is None:
        y = torch.zeros((groups, rows, H), dtype=xg.dtype, device=xg.device)
    _lib.check(_lib.load().aristos_expert_ffn_bias(_ptr(xg), _ptr(count), groups, rows, experts, _ptr(w1), _ptr(w3),
                                                   _ptr(w2), _ptr(b1), _ptr(b3), _ptr(b2), _ptr(h), _ptr(y), H, I,
                                                   hidden_act, _dt(xg) if dtype is None else dtype, row_begin, row_end,
                                                   sm_limit,
                                                   _ptr(dev_status), _stream_ptr()))
    return y


def quantize_fp8(src: torch.Tensor, block_rows: int):
    """e4m3 codes (uint8, same shape) and fp32 scales of a bf16 / fp32 tensor (..., rows, cols): block_rows 1 = per
    row and 128 columns (activations), 128 = per 128 x 128 block of every (rows, cols) matrix (weights)."""
    rows, cols = src.shape[-2], src.shape[-1]
    mats = src.numel() // (rows * cols)
    q = torch.empty(src.shape, dtype=torch.uint8, device=src.device)
    if block_rows == 1:
        scales = torch.empty((*src.shape[:-1], cols // 128), dtype=torch.float32, device=src.device)
    else:
        scales = torch.empty((*src.shape[:-2], (rows + 127) // 128, cols // 128), dtype=torch.float32,
                             device=src.device)
    _lib.check(_lib.load().aristos_quantize_fp8(_ptr(src), mats, rows, cols, block_rows, _dt(src), _ptr(q),
                                                _ptr(scales), _stream_ptr()))
    return q, scales


def expert_ffn_fp8(xq, sx, count, w1q, s1, w3q, s3, w2q, s2, hidden_act: int, dev_status=None):
    """FP8 expert FFN: xq (groups, rows, H) uint8 + sx (groups, rows, H/128); weights uint8 + block scales ->
    y (groups, rows, H) bf16."""
    groups, rows, H = xq.shape
    I = w1q.shape[1]
    dev = xq.device
    h = torch.empty((groups, rows, I), dtype=torch.bfloat16, device=dev)
    hq = torch.empty((groups, rows, I), dtype=torch.uint8, device=dev)
    sh = torch.empty((groups, rows, I // 128), dtype=torch.float32, device=dev)
    y = torch.zeros((groups, rows, H), dtype=torch.bfloat16, device=dev)
    _lib.check(_lib.load().aristos_expert_ffn_fp8(_ptr(xq), _ptr(sx), _ptr(count), groups, rows, w1q.shape[0],
                                                  _ptr(w1q), _ptr(s1), _ptr(w3q), _ptr(s3), _ptr(w2q), _ptr(s2),
                                                  _ptr(h), _ptr(hq), _ptr(sh), _ptr(y), H, I, hidden_act, 0, rows, 0,
                                                  _ptr(dev_status), _stream_ptr()))
    return y


def combine(y, slot_of, topk_w):
    S, k = slot_of.shape
    H = y.shape[-1]
    out = torch.empty((S, H), dtype=y.dtype, device=y.device)
    _lib.check(_lib.load().aristos_combine(_ptr(y), _ptr(slot_of), _ptr(topk_w), S, k, H, _dt(y), _ptr(out),
                                           _stream_ptr()))
    return out


def ffn_set_tile_mode(mode: int) -> None:
    """aristos_ffn_set_tile_mode: 0 automatic, 1 single-CTA tiles, 2 CTA pairs + single-CTA tail, 3 CTA pairs padded,
    -1 re-read ARISTOS_FFN_TILES."""
    _lib.check(_lib.load().aristos_ffn_set_tile_mode(int(mode)))


# ---- layer ----------------------------------------------------------------------------------------------------------
class MoELayer:
    """One MoE layer on the current CUDA device (aristos_moe_create ... aristos_moe_destroy)."""

    def __init__(self, cfg: AristosConfig, rank: int = 0, world: int = 1, nccl_uid: Optional[bytes] = None):
        if not torch.cuda.is_available():
            raise RuntimeError("cuplayground_b200 needs a CUDA device (sm_100a); there is no CPU fallback")
        self.cfg = cfg
        self.rank, self.world = rank, world
        self._lib = _lib.load()
        self._h = C.c_void_p()
        s = cfg.to_struct()
        uid = C.create_string_buffer(nccl_uid, 128) if nccl_uid is not None else None
        _lib.check(self._lib.aristos_moe_create(C.byref(s), rank, world, uid, C.byref(self._h)))
        self.S, self.H, self.I = cfg.S, cfg.hidden_size, cfg.intermediate_size
        self.E, self.k, self.cap = cfg.num_experts, cfg.expert_top_k, cfg.capacity
        self.E_local = self.E // world
        self.dtype = _TORCH_DTYPE[cfg.torch_dtype]
        self._ws = None

    @property
    def workspace_bytes(self) -> int:
        return int(self._lib.aristos_moe_workspace_bytes(self._h))

    def use_torch_workspace(self) -> None:
        """Allocate the workspace from torch's caching allocator instead of cudaMalloc inside the library."""
        self._ws = torch.empty(self.workspace_bytes + 1024, dtype=torch.uint8, device="cuda")
        base = (self._ws.data_ptr() + 1023) // 1024 * 1024
        _lib.check(self._lib.aristos_moe_set_workspace(self._h, C.c_void_p(base), self.workspace_bytes))

    def set_bias(self, b1=None, b3=None, b2=None) -> None:
        """Expert biases (E_local, I) / (E_local, I) / (E_local, H) for every later forward; kept alive here."""
        self._bias = (b1, b3, b2)
        _lib.check(self._lib.aristos_moe_set_bias(self._h, _ptr(b1), _ptr(b3), _ptr(b2)))

    def forward(self, x, w_gate, w1, w3, w2, gate_bias=None, out=None, stream=None, scales=None):
        """scales: fp8 only - the weights' block scales [s1 | s3 | s2] as one contiguous fp32 tensor."""
        if out is None:
            out = torch.empty_like(x)
        _lib.check(self._lib.aristos_moe_forward(self._h, _ptr(x), _ptr(w_gate), _ptr(gate_bias), _ptr(w1), _ptr(w3),
                                                 _ptr(w2), _ptr(scales), _ptr(out), _stream_ptr(stream)))
        return out

    def forward_host(self, x_host, w_gate, w1, w3, w2, out_host, gate_bias=None, stream=None, scales=None):
        """x_host / out_host: CPU tensors (pinned for full speed); weights stay on the device. Synchronous."""
        if x_host.is_cuda or out_host.is_cuda:
            raise ValueError("forward_host takes host tensors")
        _lib.check(self._lib.aristos_moe_forward_host(self._h, _ptr(x_host), _ptr(w_gate), _ptr(gate_bias), _ptr(w1),
                                                      _ptr(w3), _ptr(w2), _ptr(scales), _ptr(out_host),
                                                      _stream_ptr(stream)))
        return out_host

    def submit_host(self, x_host, w_gate, w1, w3, w2, out_host, gate_bias=None, stream=None, scales=None):
        """Asynchronous forward_host: returns once the copies and kernels are enqueued (four calls may be in flight);
        the host tensors must stay alive and untouched until wait_host()."""
        if x_host.is_cuda or out_host.is_cuda:
            raise ValueError("submit_host takes host tensors")
        _lib.check(self._lib.aristos_moe_submit_host(self._h, _ptr(x_host), _ptr(w_gate), _ptr(gate_bias), _ptr(w1),
                                                     _ptr(w3), _ptr(w2), _ptr(scales), _ptr(out_host),
                                                     _stream_ptr(stream)))

    def wait_host(self) -> None:
        _lib.check(self._lib.aristos_moe_wait_host(self._h))

    def routing(self) -> dict:
        """Host copies (CPU torch tensors) of the routing tensors of the last forward."""
        S, k, E, cap = self.S, self.k, self.E, self.cap
        idx = torch.empty((S, k), dtype=torch.int32)
        w = torch.empty((S, k), dtype=torch.float32)
        count = torch.empty(E, dtype=torch.int32)
        slot_of = torch.empty((S, k), dtype=torch.int32)
        tos = torch.empty(E * cap, dtype=torch.int32)
        _lib.check(self._lib.aristos_moe_routing_to_host(self._h, _ptr(idx), _ptr(w), _ptr(count), _ptr(slot_of),
                                                         _ptr(tos)))
        return dict(topk_idx=idx, topk_w=w, count=count, slot_of=slot_of, token_of_slot=tos, capacity=cap)

    def set_profiling(self, enable: bool) -> None:
        _lib.check(self._lib.aristos_moe_set_profiling(self._h, int(enable)))

    def stage_ms(self) -> dict:
        """Milliseconds of the stages of the last forward (profiling must be on)."""
        ms = (C.c_float * 5)()
        _lib.check(self._lib.aristos_moe_stage_ms(self._h, ms))
        return dict(gate=ms[0], dispatch=ms[1], ffn=ms[2], combine=ms[3], total=ms[4])

    def exchange_ms(self) -> float:
        """Milliseconds of the outgoing exchange (counts + gather into the peers + flags) of the last forwards."""
        ms = C.c_float(0.0)
        _lib.check(self._lib.aristos_moe_exchange_ms(self._h, C.byref(ms)))
        return float(ms.value)

    def exchange_profile(self) -> dict:
        """The expert-FFN stage of an expert-parallel layer split at its cross-rank waits (milliseconds)."""
        ms = (C.c_float * 4)()
        _lib.check(self._lib.aristos_moe_exchange_profile(self._h, ms))
        return dict(rows_sent=ms[0], counts_arrived=ms[1], gemms=ms[2], returns_arrived=ms[3])

    def status(self) -> None:
        _lib.check(self._lib.aristos_moe_status(self._h))

    def training_state(self) -> dict:
        """is_training = 1: what the last forward saved for a backward pass - host copies of the routing and the
        load-balance statistics (frac, prob per expert; aux loss; dropped share)."""
        ts = _lib.AristosTrainingStateStruct()
        _lib.check(self._lib.aristos_moe_training_state(self._h, C.byref(ts)))
        S, k, E = ts.tokens, ts.top_k, ts.num_experts
        idx = torch.empty((S, k), dtype=torch.int32)
        w = torch.empty((S, k), dtype=torch.float32)
        slot = torch.empty((S, k), dtype=torch.int32)
        lb = torch.empty(2 * E + 2, dtype=torch.float32)
        _lib.check(self._lib.aristos_moe_training_state_to_host(self._h, _ptr(idx), _ptr(w), _ptr(slot), _ptr(lb)))
        return dict(topk_idx=idx, topk_w=w, slot_of=slot, frac=lb[:E], prob=lb[E:2 * E], aux=float(lb[2 * E]),
                    dropped=float(lb[2 * E + 1]),
                    device_ptrs=(ts.topk_idx, ts.topk_w, ts.slot_of, ts.load_balance))

    def set_training_buffer(self, buf: Optional[torch.Tensor]) -> None:
        """Point the next forwards' saved training state at a caller-owned device buffer (uint8, at least
        training_bytes, 256-byte aligned); None returns to the layer's own buffer."""
        self._train_buf = buf
        if buf is None:
            _lib.check(self._lib.aristos_moe_set_training_buffer(self._h, None, 0))
        else:
            _lib.check(self._lib.aristos_moe_set_training_buffer(self._h, C.c_void_p(buf.data_ptr()), buf.numel()))

    @property
    def training_bytes(self) -> int:
        return int(self._lib.aristos_moe_training_bytes(self._h))

    def set_timeout_ms(self, timeout_ms: int) -> None:
        """Wall-clock limit of the waits for an expert-parallel forward (status, wait_host, routing, close)."""
        _lib.check(self._lib.aristos_moe_set_timeout_ms(self._h, int(timeout_ms)))

    @property
    def ep_transport(self) -> str:
        return self._lib.aristos_moe_ep_transport(self._h).decode()

    @property
    def launch_count(self) -> int:
        return int(self._lib.aristos_moe_launch_count(self._h))

    def close(self) -> None:
        if self._h:
            self._lib.aristos_moe_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
