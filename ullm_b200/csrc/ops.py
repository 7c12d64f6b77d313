"""Python face of the compiled kernels: loads the shared library with ctypes
and wraps each extern "C" launcher in a method that checks devices, dtypes,
shapes and contiguity before passing raw pointers and the current CUDA stream.

There is no CPU path here: a tensor that is not on a CUDA device is an error,
and a missing or unbuildable library is an error at first use.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .build import build

_DT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
_ERRORS = {
    1: "unsupported dtype",
    2: "bad size argument",
    3: "CUDA launch failed",
    4: "size not supported by this kernel",
}
STATUS_MESSAGES = {
    1: "token id out of range (row {index}: id {value})",
    2: "position out of range of the position table (token {index}: position {value})",
    3: "cache slot out of range (token {index}: slot {value})",
    4: "row index out of range (row {index}: {value})",
    5: "page id out of range in a block table (token {index}: page {value})",
    6: "a kernel gave up waiting on a barrier (place {index}, at {value}) and returned early",
}

MAX_HEAD_DIM = 512


class KernelError(RuntimeError):
    pass


def check_attention_sizes(num_heads: int, num_kv_heads: int, head_dim: int, rotary_dim: int) -> None:
    """Sizes the attention kernels take; anything else is refused here, at
    construction, with the reason."""
    if num_heads <= 0 or num_kv_heads <= 0 or num_heads % num_kv_heads:
        raise ValueError(f"num_heads={num_heads} must be a positive multiple of num_kv_heads={num_kv_heads}")
    if head_dim <= 0 or head_dim > MAX_HEAD_DIM:
        raise ValueError(f"head_dim={head_dim}: the attention kernels take 1..{MAX_HEAD_DIM}")
    if rotary_dim < 0 or rotary_dim > head_dim or rotary_dim % 2:
        raise ValueError(f"rotary_dim={rotary_dim} must be even and at most head_dim={head_dim}")


def _ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t: torch.Tensor, name: str, dtype=None, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}: the kernels run on CUDA tensors only (no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _timed(group: str, nbytes=None, skipped=None):
    """While a timer is installed (`Kernels.timer`, see engine/profiler.py), the wrapped call is bracketed by
    two CUDA events and booked under `group`; `nbytes(*args)` says what it had to read, if that is known.
    `skipped`: what the call returns when a measurement leaves its group out."""

    def outer(fn):
        def inner(self, *a, **k):
            if self.skip_groups and group in self.skip_groups:
                return skipped  # a measurement leaves this group out (the step's results are then meaningless)
            t = self.timer
            if t is None:
                return fn(self, *a, **k)
            start = t.begin()
            try:
                return fn(self, *a, **k)
            finally:
                t.end(group, start, nbytes(*a) if (nbytes is not None and start is not None) else 0)

        inner.__name__, inner.__doc__ = fn.__name__, fn.__doc__
        return inner

    return outer


def _weight_bytes(x, weight, *rest):
    return weight.numel() * weight.element_size()


class Kernels:
    def __init__(self, lib_path: str | None = None):
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: this engine has no CPU path")
        self.lib_path = lib_path or build()
        self.lib = ctypes.CDLL(self.lib_path)
        self._declare()
        self.status = torch.zeros(4, dtype=torch.int32, device="cuda")
        self.sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        self._f32_out_mm = None
        self._lin_ws = None  # partial sums and tile counters of the tcgen05 product, made at its first use
        self._lin_counters = None
        self.pdl = False
        self._decb = {}  # (head_dim, heads per kv head) -> (partials, prefix) of the balanced decode attention
        self._tail_ws = {}  # hidden size -> (scratch, counters) of the fused layer tail
        self.apply_switches(os.environ)
        self._lt_ok = None
        self._lt_ws = None
        self._lt_tuned = set()
        self.timer = None  # a KernelGroupTimer while a profile is being taken
        # groups of kernels (the names `_timed` books them under) that are NOT launched: only for measuring what a
        # group costs inside a step, by the difference; the step's results are wrong while this is set
        self.skip_groups: frozenset = frozenset()
        self.attention_path = None  # which attention kernel the last call chose (tests read it)
        self.launches = 0  # hand-written kernels launched (graph replays add what they captured)

    def begin_step(self, rows: int, dtype) -> None:
        """Called by the step function before a step's kernels are launched (or recorded into a CUDA graph): with
        the automatic policy, programmatic dependent launch is on for exactly the steps whose products are all the
        stream kernel (bfloat16, at most `stream_all_rows` rows), and off otherwise."""
        if self.pdl_mode == "auto":
            self.set_pdl(bool(dtype == torch.bfloat16 and self.small_m_mode == "auto" and rows <= self.stream_all_rows))

    # -- switches -----------------------------------------------------------
    SWITCHES = ("ULLM_B200_PDL", "ULLM_B200_DECODE_SPLIT_TARGET", "ULLM_B200_TC_ATTN", "ULLM_B200_DECODE_CLUSTER",
                "ULLM_B200_FUSE_DECODE_ROPE", "ULLM_B200_MIXED_DECODE_ROWS", "ULLM_B200_DECODE_TC",
                "ULLM_B200_DECODE_BALANCED", "ULLM_B200_SMALL_M_LINEAR", "ULLM_B200_STREAM_WEIGHT_MB",
                "ULLM_B200_FUSED_MLP_ROWS", "ULLM_B200_LT_ROWS", "ULLM_B200_FUSED_TAIL_ROWS",
                "ULLM_B200_STREAM_ALL_ROWS", "ULLM_B200_CHAIN_NORMS", "ULLM_B200_GENERAL_ATTN_TC")

    def apply_switches(self, env) -> None:
        """Sets every kernel choice from `env` (a mapping; the process environment at start-up): a switch that is
        not in it takes its default.  All switches are optional; the defaults are what was measured fastest."""
        get = env.get
        # programmatic dependent launch for every kernel of the library: "auto" (the default) for the steps whose
        # products are all the stream kernel (see `begin_step`), where its ring fills with weights while the kernel
        # in front drains (Qwen3-8B sizes, batch 1: 3.60 -> 3.38 ms per step); "1" always, "0" never (with the
        # library's products in between it costs 1 to 2 %: waiting blocks hold SM slots and gain nothing)
        mode = get("ULLM_B200_PDL", "auto")
        self.pdl_mode = {"1": True, "0": False}.get(mode, "auto")
        self.set_pdl(self.pdl_mode is True)
        # blocks the per-request decode attention aims for when it splits the requests' key ranges
        self.decode_split_target = int(get("ULLM_B200_DECODE_SPLIT_TARGET", "400"))
        # prompt attention on the tcgen05 tensor cores (head size 128); 0: the mma.sync kernel
        # prompt attention at head size 128: "1" the tcgen05 kernels (two query tiles per block where a request
        # brings more than one tile, else one), "pair" / "single" one of them always, "0" the mma.sync kernel
        self.tc_attention_mode = get("ULLM_B200_TC_ATTN", "1")
        self.use_tcgen05_attention = self.tc_attention_mode != "0"
        # attention with capped scores or mixed heads (the general path of parts/attention.py) on the tensor-core
        # kernels where the sizes allow; 0: the general kernel always
        self.general_attention_tc = get("ULLM_B200_GENERAL_ATTN_TC", "1") != "0"
        # windowed attention with its further options (values inside the keys, slopes, pooled blocks, a gate) on the
        # tensor-core kernel of csrc/attention_window.cu where the sizes allow; 0: the general kernel always
        self.window_attention_tc = get("ULLM_B200_WINDOW_ATTN_TC", "1") != "0"
        # the splits of a request's keys merge inside a thread-block cluster (at most 8 splits) instead of through
        # scratch arrays and a second kernel
        # ("auto": for steps of at most 8 rows; "1" / "0": always / never, with `decode_split_target` splits)
        mode = get("ULLM_B200_DECODE_CLUSTER", "auto")
        self.decode_cluster_merge = {"1": True, "0": False}.get(mode, "auto")
        # decode steps: the per-request decode attention kernel applies the q/k norm and the rotation and writes the
        # new key and value itself (one launch less per layer)
        self.fuse_decode_rope = get("ULLM_B200_FUSE_DECODE_ROPE", "1") == "1"
        # a mixed step's leading one-token entries go to the decode attention kernel from this many on (0: never)
        self.mixed_decode_rows = int(get("ULLM_B200_MIXED_DECODE_ROWS", "4"))
        # decode attention on the tcgen05 tensor cores (head size 128), the batch's keys cut evenly over the blocks
        self.use_tcgen05_decode = get("ULLM_B200_DECODE_TC", "0") == "1"
        # decode attention: the batch's keys cut evenly over the warps (True), every request split alike (False),
        # or "auto": the first for batches of very unequal lengths (the mixer says so), else the second
        mode = get("ULLM_B200_DECODE_BALANCED", "auto")
        self.use_balanced_decode = {"1": True, "0": False}.get(mode, "auto")
        # few-row products: "auto" (the default) the weight-streaming TMA kernel for small weights, where a step is
        # bound by launches and start-up and not by memory (measured at Qwen3-0.6B sizes: a decode step of 4 to 16
        # requests 6 to 17 % faster), the library otherwise; "0" always the library; "stream" that kernel always
        # (M <= 32), "skinny" the mma.sync streaming kernel (M <= 32), "tcgen05" (or "1") the stream-K tcgen05
        # kernel (M <= 64)
        mode = get("ULLM_B200_SMALL_M_LINEAR", "auto")
        self.small_m_mode = {"1": "tcgen05", "0": None, "": "auto"}.get(mode, mode)
        # "auto": rows up to which EVERY product of a step is the stream kernel (with dependent launch it beats
        # the library there: Qwen3-8B sizes, 8 requests 4.14 -> 3.60 ms per step, 1 request 3.63 -> 3.32, 16 requests
        # 4.68 -> 4.58)
        self.stream_all_rows = int(get("ULLM_B200_STREAM_ALL_ROWS", "16"))
        # in those steps a block folds its feed-forward norm between the output projection and the gate / up
        # product (one kernel less per layer); 0: the norm stays a kernel of its own
        # 0: norms stay kernels of their own; 1: a block's feed-forward norm is folded between its products in
        # small decode steps; 2: the next block's first norm too (behind this block's last product)
        self.chain_norms = int(get("ULLM_B200_CHAIN_NORMS", "2"))
        if self.small_m_mode not in (None, "auto", "tcgen05", "skinny", "stream"):
            raise KernelError(f"ULLM_B200_SMALL_M_LINEAR={mode!r}: auto, 0, stream, skinny or tcgen05")
        self.stream_weight_bytes = int(get("ULLM_B200_STREAM_WEIGHT_MB", "16")) << 20  # "auto": weights up to this
        self.stream_rows = 32  # rows the stream product takes
        # rows from which the gated feed-forward's first product runs on the own tcgen05 kernel with the activation
        # fused (0 rows would mean always; a huge number never)
        self.fused_mlp_rows = int(get("ULLM_B200_FUSED_MLP_ROWS", "4096"))
        # rows up to which the library's product is called through cuBLASLt with a timed choice of algorithm
        self.lt_rows = int(get("ULLM_B200_LT_ROWS", str(1 << 30)))
        # rows up to which a step runs the second half of a layer (output projection, residual, norm, gated
        # feed-forward, residual) as one cooperative kernel; 0 (the default): never.  Measured at Qwen3-8B sizes:
        # 71 us against 70 us for the separate kernels at 8 rows, 77 against 70 at 16: no gain yet.
        self.fused_tail_rows = int(get("ULLM_B200_FUSED_TAIL_ROWS", "0"))

    # -- ctypes signatures --------------------------------------------------
    def _declare(self) -> None:
        L = self.lib
        P, I, F, LL = c_void_p, c_int, c_float, c_longlong
        sig = {
            "ullm_embedding": [I, P, P, P, I, I, I, P, P, P, P, P],
            "ullm_gather_rows": [I, P, P, P, I, I, I, P, P],
            "ullm_add_rmsnorm": [I, P, P, P, P, I, I, F, P],
            "ullm_act_mul": [I, I, P, P, I, I, P],
            "ullm_cast_bf16_f32": [P, P, LL, P],
            "ullm_qk_norm_rope_store": [I, P, I, I, I, I, P, P, F, P, P, I, I, P, P, P, P, LL, P, P],
            "ullm_qk_norm_in_place": [I, P, I, I, I, I, P, P, F, P, P],
            "ullm_paged_attention_generic": [I, P, LL, P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, F, LL, P, P],
            "ullm_decode_attention": [P, LL, P, P, P, I, P, P, P, P, I, I, I, I, I, I, F, I, LL, P, P],
            "ullm_decode_attention_balanced": [P, LL, P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, F, LL, P, P],
            "ullm_decode_attention_fused": [P, LL, P, P, P, I, P, P, P, P, I, I, I, I, I, I, F, I, LL, P, P, F, P, P, I,
                                            P, P, P, P],
            "ullm_prefill_attention": [P, LL, P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, LL, P, P],
            "ullm_prefill_attention_kept": [P, LL, P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, LL, P, P, I],
            "ullm_decode_attention_kept": [P, LL, P, P, P, I, P, P, P, P, I, I, I, I, I, I, F, I, LL, P, P, I],
            "ullm_decode_attention_capped": [P, LL, P, P, P, I, P, P, P, P, I, I, I, I, I, I, F, I, LL, P, P, I, F],
            "ullm_decode_attention_parts": [P, LL, P, P, P, I, P, P, P, P, I, I, I, I, I, I, F, I, LL, P, P, I],
            "ullm_prefill_attention_ex": [P, LL, P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, LL, P, P, I, F, P],
            "ullm_prefill_attention_tcgen05": [P, LL, P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, LL, P, P],
            "ullm_prefill_attention_pair": [P, LL, P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, LL, P, P],
            "ullm_prefill_attention_pair_capped": [P, LL, P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, LL, P, P, F],
            "ullm_prefill_attention_pair_parts": [P, LL, P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, LL, P, P],
            "ullm_linear_tcgen05": [P, P, P, P, I, I, I, I, I, P, LL, P, I, P, P],
            "ullm_linear_skinny": [P, P, P, P, I, I, I, I, I, P],
            "ullm_linear_stream": [P, P, P, P, P, I, I, I, I, I, P, P],
            "ullm_linear_stream_norm": [P, P, P, P, P, I, I, I, I, I, P, P, P, P, I, I, F, P, P],
            "ullm_layer_tail_fused": [P, P, P, P, P, P, P, P, F, I, I, I, I, I, P, P, P, P],
            "ullm_linear_tcgen05_large": [P, P, P, P, I, I, I, I, I, I, P, P],
            "ullm_decode_attention_tcgen05": [P, LL, P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, F, LL, P, P],
            "ullm_lt_linear": [P, P, P, I, I, I, I, P, LL, I, P, LL, P],
            "ullm_paged_attention_generic_ex": [I, P, LL, P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, F, LL, P, P, I, I],
            "ullm_qk_norm_rope_store_ex": [I, P, I, I, I, I, P, P, F, P, P, I, I, P, P, P, P, LL, P, P, I, I],
            "ullm_act_mul_clamped": [I, P, P, I, I, F, F, P],
            "ullm_embed_scaled": [I, P, P, P, P, I, I, I, F, P, P, P, P, P, P, P],
            "ullm_norm_scale_add": [I, P, P, P, P, I, I, F, F, P],
            "ullm_norm_scale_add_norm": [I, P, P, P, I, I, F, F, P, F, P, P],
            "ullm_rmsnorm_rows_f32": [I, P, P, P, P, I, I, I, F, P, P],
            "ullm_cast_rows_f32": [I, P, P, LL, P],
            "ullm_mlstm_recurrence": [I, P, LL, I, I, I, P, P, P, P, LL, P, P, P, P, I, I, I, I, F, F, I, P, P],
            "ullm_mlstm_out_gate": [I, P, P, LL, P, P, I, I, I, F, P],
            "ullm_gated_add_f32": [I, P, P, P, LL, P, P, P, P, I, I, P],
            "ullm_side_gate_mul": [I, P, P, P, LL, I, P, I, I, I, P, P, P, P, P],
            "ullm_softcap_f32": [P, LL, F, P],
            "ullm_qkv_prepare": [I, P, LL, I, I, I, I, I, P, I, P, LL, P, P, P, I, P, P, I, P, P, I, I, F, I, P, P, P, P,
                                 P, LL, P, P, P],
            "ullm_conv_state_update": [I, P, LL, I, I, P, LL, P, P, P, I, I, P],
            "ullm_paged_attention_generic_ex2": [I, P, LL, P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, F, LL, P, P, I, I,
                                                 F, P],
            "ullm_mix_heads": [I, P, P, P, I, I, I, I, P],
            "ullm_window_attention": [P, LL, P, LL, P, P, P, I, P, P, P, I, I, I, I, I, I, I, I, F, LL, P, P, P, I, P, P,
                                      P, I, LL, P, LL, F, I, P],
            "ullm_paged_attention_generic_ex3": [I, P, LL, P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, F, LL, P, P, I, I,
                                                 F, P, I, I, P, P, P, I, LL, P, LL, F, LL],
            "ullm_norm_add_norm": [I, P, P, P, I, I, F, F, I, P, P, P, F, I, I, P, P],
            "ullm_norm_rows": [I, P, P, P, P, I, I, I, F, I, P, P],
            "ullm_xielu": [I, P, P, LL, P, P],
            "ullm_kv_shared_prepare": [I, P, LL, I, I, I, P, P, F, P, P, P, LL, P, P],
            "ullm_pool_blocks": [I, P, P, P, P, I, I, LL, P, P, I, I, P, LL, P, P, I, I, P, P],
            "ullm_latent_prepare": [I, P, P, P, P, I, I, I, I, I, I, P, F, P, P, P, P, LL, P, P, I, LL, LL],
            "ullm_qkv_rows_prepare": [I, P, LL, P, I, I, I, I, I, P, P, F, P, I, I, P, P, I, P, P, P, LL, P, P],
            "ullm_concat_rows_f32": [I, P, P, P, I, I, I, P],
            "ullm_sigmoid_gate": [I, P, P, LL, I, I, P],
            "ullm_mingru": [I, P, LL, I, I, I, P, P, P, LL, P, P, P, P, LL, F, I, I, I, P, P],
            "ullm_gla_recurrence": [I, P, LL, I, I, I, P, LL, P, F, F, P, LL, P, P, P, P, I, I, I, I, I, I, P, P],
            "ullm_head_norm_gate": [I, P, P, LL, P, P, I, I, I, F, I, I, P],
            "ullm_moe_route": [P, LL, P, P, P, I, I, I, I, I, P],
            "ullm_moe_arrange": [P, I, I, P, P, P, P],
            "ullm_moe_grouped_linear": [I, P, LL, P, LL, P, P, P, P, I, I, I, I, I, I, I, I, F, F, P],
            "ullm_moe_combine": [I, P, P, P, P, I, I, I, P, I, P, LL, P, P, LL, P],
            "ullm_moe_combine_add_norm": [I, P, P, P, I, I, I, P, I, P, LL, P, P, LL, P, P, P, F, P, P],
            "ullm_argmax": [P, LL, I, I, P, P],
            "ullm_sample": [P, LL, I, I, P, P, P, P, P, P, P, P, P, P],
        }
        for name, args in sig.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = c_int
        L.ullm_mingru_chunk.argtypes = []
        L.ullm_mingru_chunk.restype = c_int
        L.ullm_moe_force_plain.argtypes = [I]
        L.ullm_moe_force_plain.restype = None
        L.ullm_mlstm_supported.argtypes = [I, I, I]
        L.ullm_mlstm_supported.restype = c_int
        L.ullm_mlstm_state_floats.argtypes = [I, I, I]
        L.ullm_mlstm_state_floats.restype = c_longlong
        L.ullm_gla_supported.argtypes = [I, I, I]
        L.ullm_gla_supported.restype = c_int
        L.ullm_gla_state_floats.argtypes = [I, I, I]
        L.ullm_gla_state_floats.restype = c_longlong
        L.ullm_wait_selftest.argtypes = [I, P, P, P]
        L.ullm_wait_selftest.restype = c_int
        L.ullm_decode_attention_supported.argtypes = [I, I, I]
        L.ullm_decode_attention_supported.restype = c_int
        L.ullm_decode_attention_balanced_supported.argtypes = [I, I, I, I, I]
        L.ullm_decode_attention_balanced_supported.restype = c_int
        L.ullm_decode_attention_balanced_scratch_floats.argtypes = [I, I]
        L.ullm_decode_attention_balanced_scratch_floats.restype = c_longlong
        L.ullm_decode_attention_tcgen05_supported.argtypes = [I, I, I, I, I]
        L.ullm_decode_attention_tcgen05_supported.restype = c_int
        L.ullm_decode_attention_tcgen05_scratch_floats.argtypes = [I]
        L.ullm_decode_attention_tcgen05_scratch_floats.restype = c_longlong
        L.ullm_decode_attention_cluster_merge.argtypes = [I]
        L.ullm_decode_attention_cluster_merge.restype = None
        L.ullm_decode_attention_last_used_cluster.argtypes = []
        L.ullm_decode_attention_last_used_cluster.restype = c_int
        L.ullm_sample_force_one_block.argtypes = [I]
        L.ullm_sample_force_one_block.restype = None
        L.ullm_sample_last_used_cluster.argtypes = []
        L.ullm_sample_last_used_cluster.restype = c_int
        L.ullm_lt_available.argtypes = []
        L.ullm_lt_available.restype = c_int
        L.ullm_lt_last_choice.argtypes = [P, P, P, P]
        L.ullm_lt_last_choice.restype = None
        L.ullm_window_attention_supported.argtypes = [I, I, I, I, I]
        L.ullm_window_attention_supported.restype = c_int
        L.ullm_prefill_attention_supported.argtypes = [I, I, I]
        L.ullm_prefill_attention_supported.restype = c_int
        L.ullm_prefill_attention_tcgen05_supported.argtypes = [I, I, I, I]
        L.ullm_prefill_attention_tcgen05_supported.restype = c_int
        L.ullm_prefill_attention_tcgen05_blocks_per_sm.restype = c_int
        L.ullm_prefill_attention_pair_supported.argtypes = [I, I, I, I]
        L.ullm_prefill_attention_pair_supported.restype = c_int
        L.ullm_set_pdl.argtypes = [I]
        L.ullm_set_pdl.restype = None
        L.ullm_linear_tcgen05_supported.argtypes = [I, I, I]
        L.ullm_linear_tcgen05_supported.restype = c_int
        L.ullm_linear_tcgen05_blocks.restype = c_int
        L.ullm_linear_tcgen05_large_supported.argtypes = [I, I, I]
        L.ullm_linear_tcgen05_large_supported.restype = c_int
        L.ullm_linear_skinny_supported.argtypes = [I, I, I]
        L.ullm_linear_skinny_supported.restype = c_int
        L.ullm_layer_tail_fused_supported.argtypes = [I, I, I, I]
        L.ullm_layer_tail_fused_supported.restype = c_int
        L.ullm_layer_tail_fused_scratch_floats.argtypes = [I]
        L.ullm_layer_tail_fused_scratch_floats.restype = c_longlong
        L.ullm_layer_tail_fused_counters.argtypes = [I]
        L.ullm_layer_tail_fused_counters.restype = c_longlong
        L.ullm_layer_tail_fused_last_grid.restype = c_int
        L.ullm_linear_stream_supported.argtypes = [I, I, I]
        L.ullm_linear_stream_supported.restype = c_int
        L.ullm_linear_stream_sq_floats.argtypes = [I]
        L.ullm_linear_stream_sq_floats.restype = c_longlong
        L.ullm_linear_stream_blocks_per_sm.argtypes = [I]
        L.ullm_linear_stream_blocks_per_sm.restype = None
        L.ullm_linear_stream_smem_kb.argtypes = [I]
        L.ullm_linear_stream_smem_kb.restype = None
        L.ullm_linear_stream_ksplit_max.argtypes = [I]
        L.ullm_linear_stream_ksplit_max.restype = None

    def _check(self, code: int, what: str) -> None:
        self.launches += 1
        if code != 0:
            raise KernelError(f"{what}: {_ERRORS.get(code, f'error {code}')}")

    def set_pdl(self, on: bool) -> None:
        """Programmatic dependent launch for every kernel of the library: a kernel's launch and
        set-up overlap the tail of the kernel before it in the stream."""
        if bool(on) != self.pdl:
            self.lib.ullm_set_pdl(1 if on else 0)
            self.pdl = bool(on)

    # -- status word ----------------------------------------------------------
    def raise_on_status(self) -> None:
        """Reads the device status word (synchronizes) and raises if a kernel
        refused an out-of-range index since the last call."""
        s = self.status.tolist()
        if s[0] != 0:
            self.status.zero_()
            if self._lin_counters is not None:
                self._lin_counters.zero_()  # a product that gave up may have left tiles half counted
            for _part, _prefix, flags in self._decb.values():
                flags.zero_()  # likewise the merge flags of the balanced decode attention
            for _scratch, counters, _normed in self._tail_ws.values():
                counters.zero_()  # and the tickets and grid barriers of the fused layer tail
            msg = STATUS_MESSAGES.get(s[0], "status {code}").format(index=s[1], value=s[2], code=s[0])
            raise KernelError(f"a kernel refused an index: {msg}")

    def wait_selftest(self, limit: int = 4096) -> int:
        """Runs the kernels' give-up path on purpose (see csrc/wait_selftest.cu): a one-block kernel waits
        `limit` polls on a barrier nobody arrives at, records the timeout in the status word, frees its tensor
        memory and returns.  Returns 1 when the wait ran out; the status word is left set for the caller
        (`raise_on_status` reads and clears it)."""
        out = torch.zeros(1, dtype=torch.int32, device="cuda")
        self._check(self.lib.ullm_wait_selftest(int(limit), _ptr(self.status), _ptr(out), _stream()), "wait_selftest")
        return int(out.item())

    # -- library matrix products ---------------------------------------------
    def small_m_linear(self, x, weight, out, bias=None, act: int | None = None) -> bool:
        """The hand-written tcgen05/TMA product for few rows (decode steps): bfloat16 operands, out bfloat16
        or float32; with `act` (0 silu, 1 gelu_tanh) weight stacks gate rows on up rows and out is
        act(gate) * up.  False when the shape is not one it takes (the caller then uses the library)."""
        M, K = x.shape
        N = weight.shape[0]
        n_out = N // 2 if act is not None else N
        if (x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not x.is_contiguous()
                or not weight.is_contiguous() or not out.is_contiguous() or weight.shape[1] != K
                or out.shape != (M, n_out) or out.dtype not in (torch.bfloat16, torch.float32)
                or (bias is not None and bias.dtype != torch.bfloat16) or (act is not None and N % 2)
                or not self.lib.ullm_linear_tcgen05_supported(M, N, K)
                or x.data_ptr() % 16 or weight.data_ptr() % 16):
            return False
        if self._lin_ws is None:
            blocks = self.lib.ullm_linear_tcgen05_blocks()
            if blocks <= 0:
                raise KernelError("linear_tcgen05: cannot read the device's SM count")
            self._lin_ws = torch.empty(blocks * 2 * 64 * 128, dtype=torch.float32, device="cuda")
            self._lin_counters = torch.zeros(16384, dtype=torch.int32, device="cuda")
        code = self.lib.ullm_linear_tcgen05(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), M, N, K,
                                            1 if out.dtype == torch.float32 else 0, 0 if act is None else act + 1,
                                            _ptr(self._lin_ws), self._lin_ws.numel(), _ptr(self._lin_counters),
                                            self._lin_counters.numel(), _ptr(self.status), _stream())
        if code == 4:  # more tiles than counters: the library takes it
            return False
        self._check(code, f"linear_tcgen05 ({M}x{K} . {N}x{K})")
        return True

    def skinny_linear(self, x, weight, out, bias=None, act: int | None = None) -> bool:
        """The streaming mma.sync product for very few rows (M <= 32), same contract as `small_m_linear`."""
        M, K = x.shape
        N = weight.shape[0]
        n_out = N // 2 if act is not None else N
        if (x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not x.is_contiguous()
                or not weight.is_contiguous() or not out.is_contiguous() or weight.shape[1] != K
                or out.shape != (M, n_out) or out.dtype not in (torch.bfloat16, torch.float32)
                or (bias is not None and bias.dtype != torch.bfloat16) or (act is not None and N % 2)
                or not self.lib.ullm_linear_skinny_supported(M, N, K)
                or x.data_ptr() % 16 or weight.data_ptr() % 16):
            return False
        self._check(self.lib.ullm_linear_skinny(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), M, N, K,
                                                1 if out.dtype == torch.float32 else 0,
                                                0 if act is None else act + 1, _stream()),
                    f"linear_skinny ({M}x{K} . {N}x{K})")
        return True

    @_timed("linear", _weight_bytes, skipped=True)
    def stream_linear(self, x, weight, out, bias=None, act: int | None = None, residual=None, norm_behind=None,
                      norm_in_front=None) -> bool:
        """`_stream_linear` as a call of its own (a block that chains its products): booked under the products'
        group."""
        return self._stream_linear(x, weight, out, bias, act, residual, norm_behind, norm_in_front)

    def _stream_linear(self, x, weight, out, bias=None, act: int | None = None, residual=None, norm_behind=None,
                       norm_in_front=None) -> bool:
        """The weight-streaming product for few rows (M <= 32; csrc/linear_stream.cu): a TMA ring per block that
        is filled with weight tiles before the kernel in front has finished (programmatic dependent launch),
        mma.sync on the swizzled tiles.  Same contract as `small_m_linear`; `residual` ([M, n_out], bfloat16;
        may be `out`) is added to the product in 32-bit before the one rounding.

        An RMSNorm between two such products costs no kernel (rmsnorm(r) * w = (1 / rms(r)) * (r * w)):
        `norm_behind=(w, operand, sq)` on the product in front of the norm also writes result * w to `operand`
        ([M, n_out] bfloat16) and the units' sums of squares to `sq` (float32, `stream_sq_floats(n_out)`);
        `norm_in_front=(sq, cols, eps)` on the product behind it (whose x is that operand) multiplies its sums by
        the rows' 1 / rms.  Both for at most 16 rows."""
        M, K = x.shape
        N = weight.shape[0]
        n_out = N // 2 if act is not None else N
        if (x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not x.is_contiguous()
                or not weight.is_contiguous() or not out.is_contiguous() or weight.shape[1] != K
                or out.shape != (M, n_out) or out.dtype not in (torch.bfloat16, torch.float32)
                or (bias is not None and bias.dtype != torch.bfloat16) or (act is not None and N % 2)
                or (residual is not None and (residual.dtype != torch.bfloat16 or residual.shape != (M, n_out)
                                              or not residual.is_contiguous()))
                or not self.lib.ullm_linear_stream_supported(M, N, K)
                or x.data_ptr() % 16 or weight.data_ptr() % 16):
            return False
        pre_w = pre_out = sq_out = sq_in = None
        sq_count, sq_cols, sq_eps = 0, 0, 0.0
        if norm_behind is not None:
            pre_w, pre_out, sq_out = norm_behind
            _need(pre_w, "norm weight", torch.float32)
            _need(pre_out, "normed operand", torch.bfloat16)
            _need(sq_out, "sums of squares", torch.float32)
            if (act is not None or M > 16 or pre_w.numel() != n_out or pre_out.shape != (M, n_out)
                    or sq_out.numel() < self.stream_sq_floats(n_out)):
                raise KernelError("stream_linear: norm_behind needs a plain product of at most 16 rows, a weight per "
                                  "output column, an operand of the output's shape and room for the sums of squares")
        if norm_in_front is not None:
            sq_in, sq_cols, sq_eps = norm_in_front
            _need(sq_in, "sums of squares", torch.float32)
            if M > 16 or sq_cols != K or sq_in.numel() < self.stream_sq_floats(K):
                raise KernelError("stream_linear: norm_in_front needs at most 16 rows and the sums of squares of K columns")
            sq_count = self.stream_sq_floats(K) // 16
        self._check(self.lib.ullm_linear_stream_norm(
            _ptr(x), _ptr(weight), _ptr(bias), _ptr(residual), _ptr(out), M, N, K, 1 if out.dtype == torch.float32 else 0,
            0 if act is None else act + 1, _ptr(pre_w), _ptr(pre_out), _ptr(sq_out), _ptr(sq_in), sq_count, int(sq_cols),
            float(sq_eps), _ptr(self.status), _stream()), f"linear_stream ({M}x{K} . {N}x{K})")
        return True

    def stream_sq_floats(self, n_out: int) -> int:
        """Floats of the sums-of-squares array that `stream_linear(norm_behind=...)` fills for `n_out` columns."""
        return int(self.lib.ullm_linear_stream_sq_floats(int(n_out)))

    def stream_chain_applies(self, rows: int, dtype) -> bool:
        """True for the steps whose products are all the stream kernel (the automatic policy, bfloat16, few rows):
        a block may then chain its products with the norm folded between them."""
        return bool(self.small_m_mode == "auto" and dtype == torch.bfloat16 and rows <= min(self.stream_all_rows, 16)
                    and self.chain_norms > 0)

    def layer_tail_applies(self, rows: int, dtype, hidden: int, attn_width: int, intermediate: int) -> bool:
        """True when `fused_layer_tail` takes these sizes and the switch is on: decode-sized batches (at most
        `fused_tail_rows` rows, never more than 16) in bfloat16."""
        return bool(self.fused_tail_rows > 0 and rows <= min(self.fused_tail_rows, 16) and dtype == torch.bfloat16
                    and self.lib.ullm_layer_tail_fused_supported(rows, hidden, attn_width, intermediate))

    @_timed("layer_tail_fused", lambda self_attn, residual, act_out, w_o, w_gate_up, w_down, *r: (
        w_o.numel() + w_gate_up.numel() + w_down.numel()) * 2)
    def fused_layer_tail(self, attn, residual, act_out, w_o, w_gate_up, w_down, norm_w, eps: float, act: int = 0):
        """The second half of a pre-norm decoder layer in one kernel (csrc/layer_tail_fused.cu):
        residual += attn @ w_o.T;  act_out = act(h @ Wgate.T) * (h @ Wup.T) with h = rmsnorm(residual) * norm_w;
        residual += act_out @ w_down.T.  `residual` [M, H] is updated in place; `act_out` [M, I] is a work buffer.
        bfloat16, M <= 16.  Call `layer_tail_applies` first."""
        M, QD = attn.shape
        H = residual.shape[1]
        inter = act_out.shape[1]
        for t_, n_ in ((attn, "attn"), (residual, "residual"), (act_out, "act_out"), (w_o, "w_o"),
                       (w_gate_up, "w_gate_up"), (w_down, "w_down")):
            _need(t_, n_, torch.bfloat16)
            if t_.data_ptr() % 16:
                raise KernelError(f"fused_layer_tail: {n_} is not 16-byte aligned")
        _need(norm_w, "norm_w", torch.float32)
        if (residual.shape[0] != M or act_out.shape[0] != M or w_o.shape != (H, QD) or w_gate_up.shape != (2 * inter, H)
                or w_down.shape != (H, inter) or norm_w.numel() != H):
            raise KernelError(f"fused_layer_tail: attn {tuple(attn.shape)}, residual {tuple(residual.shape)}, act_out "
                              f"{tuple(act_out.shape)}, w_o {tuple(w_o.shape)}, w_gate_up {tuple(w_gate_up.shape)}, "
                              f"w_down {tuple(w_down.shape)}")
        ws = self._tail_ws.get(H)
        if ws is None:  # scratch of the split units and the zeroed counters, made at the first (eager) call
            ws = (torch.empty(self.lib.ullm_layer_tail_fused_scratch_floats(H), dtype=torch.float32, device="cuda"),
                  torch.zeros(self.lib.ullm_layer_tail_fused_counters(H), dtype=torch.int32, device="cuda"),
                  torch.empty(16, H, dtype=torch.bfloat16, device="cuda"))  # the normed rows between its phases
            self._tail_ws[H] = ws
        self._check(self.lib.ullm_layer_tail_fused(
            _ptr(attn), _ptr(residual), _ptr(act_out), _ptr(ws[2]), _ptr(w_o), _ptr(w_gate_up), _ptr(w_down), _ptr(norm_w),
            float(eps), act + 1, M, H, QD, inter, _ptr(ws[0]), _ptr(ws[1]), _ptr(self.status), _stream()),
            f"layer_tail_fused ({M} rows, hidden {H}, intermediate {inter})")
        return residual

    def large_linear(self, x, weight, out, bias=None, act: int | None = None, variant: int = 0) -> bool:
        """The persistent tcgen05/TMA product for many rows (prompt portions): tiles of 128 x 256, two accumulators
        in tensor memory, bias and the gate activation in the epilogue.  Same contract as `small_m_linear`."""
        M, K = x.shape
        N = weight.shape[0]
        n_out = N // 2 if act is not None else N
        if (x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not x.is_contiguous()
                or not weight.is_contiguous() or not out.is_contiguous() or weight.shape[1] != K
                or out.shape != (M, n_out) or out.dtype not in (torch.bfloat16, torch.float32)
                or (bias is not None and bias.dtype != torch.bfloat16) or (act is not None and N % 2)
                or not self.lib.ullm_linear_tcgen05_large_supported(M, N, K)
                or x.data_ptr() % 16 or weight.data_ptr() % 16 or out.data_ptr() % 16):
            return False
        self._check(self.lib.ullm_linear_tcgen05_large(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), M, N, K,
                                                       1 if out.dtype == torch.float32 else 0,
                                                       0 if act is None else act + 1, variant, _ptr(self.status),
                                                       _stream()),
                    f"linear_tcgen05_large ({M}x{K} . {N}x{K})")
        return True

    def lt_linear(self, x, weight, out, tune: bool = True) -> bool:
        """out = x @ weight.T through cuBLASLt with a measured choice among the library's candidate algorithms
        (timed once per shape, outside stream captures, with L2 flushed; kept for the life of the process).
        bfloat16 operands, bfloat16 or float32 out, no bias.  False: not taken (the caller uses torch)."""
        M, K = x.shape
        N = weight.shape[0]
        if (x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not x.is_contiguous()
                or not weight.is_contiguous() or not out.is_contiguous() or weight.shape[1] != K
                or out.shape != (M, N) or out.dtype not in (torch.bfloat16, torch.float32) or K % 8
                or (out.dtype == torch.bfloat16 and N % 8)
                or x.data_ptr() % 16 or weight.data_ptr() % 16 or out.data_ptr() % 16):
            return False
        if self._lt_ok is None:
            self._lt_ok = bool(self.lib.ullm_lt_available())
            if self._lt_ok:
                self._lt_ws = torch.empty(32 << 20, dtype=torch.uint8, device="cuda")
        if not self._lt_ok:
            return False
        out_f32 = 1 if out.dtype == torch.float32 else 0
        key = (M, N, K, out_f32)
        flush = None
        if tune and key not in self._lt_tuned and not torch.cuda.is_current_stream_capturing():
            try:
                flush = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda")  # larger than L2; gone after this call
            except torch.cuda.OutOfMemoryError:
                flush = None  # no room to time anything: the library's first candidate it is
            self._lt_tuned.add(key)
        rc = self.lib.ullm_lt_linear(_ptr(x), _ptr(weight), _ptr(out), M, N, K, out_f32, _ptr(self._lt_ws),
                                     self._lt_ws.numel(), 1 if flush is not None else 0, _ptr(flush),
                                     0 if flush is None else flush.numel(), _stream())
        if rc == 4:  # a shape the library has no candidate for
            return False
        self._check(rc, f"lt_linear ({M}x{K} . {N}x{K})")
        return True

    def _lt_takes(self, rows: int, weight) -> bool:
        """Products that go through the timed choice: weights of at least 8 MB (below that there is nothing to
        gain and a timing pass per shape to lose) at the padded row counts of decode steps (1, 2, 4, 8, 16, 32, 48,
        64) and at whole multiples of 256 rows (full prompt portions).  Other row counts would each cost a timing pass for a shape that may
        never come again; they take the library's own first choice."""
        if rows > self.lt_rows or weight.numel() < (1 << 22):
            return False
        return rows in (1, 2, 4, 8) or rows % 16 == 0 and (rows <= 64 or rows % 256 == 0)

    def lt_last_choice(self) -> dict:
        """The last timed choice: index in the library's list, candidates, microseconds (chosen, list's first)."""
        c, n = c_int(0), c_int(0)
        b, f = c_float(0), c_float(0)
        self.lib.ullm_lt_last_choice(ctypes.byref(c), ctypes.byref(n), ctypes.byref(b), ctypes.byref(f))
        return {"chosen": c.value, "candidates": n.value, "best_us": b.value, "first_us": f.value}

    def _own_linear(self, x, weight, out, bias=None, act=None) -> bool:
        """Tries the hand-written few-row product that the mode names; False: the caller uses the library."""
        if self.small_m_mode == "skinny":
            return x.shape[0] <= 32 and self.skinny_linear(x, weight, out, bias, act)
        if self.small_m_mode == "stream":
            return x.shape[0] <= self.stream_rows and self._stream_linear(x, weight, out, bias, act)
        if self.small_m_mode == "auto":
            rows = x.shape[0]
            return (rows <= self.stream_rows
                    and (rows <= self.stream_all_rows
                         or weight.numel() * weight.element_size() <= self.stream_weight_bytes)
                    and self._stream_linear(x, weight, out, bias, act))
        if self.small_m_mode == "tcgen05":
            if x.shape[0] <= 64:
                return self.small_m_linear(x, weight, out, bias, act)
            return self.large_linear(x, weight, out, bias, act)
        return False

    @_timed("linear", _weight_bytes)
    def linear(self, x, weight, out, bias=None):
        """out = x @ weight.T (+ bias).  Few bfloat16 rows: a hand-written kernel when one is switched on.
        Otherwise the vendor library's matrix product, float32 without any reduced-precision mode."""
        _need(x, "x")
        _need(out, "out")
        if self._own_linear(x, weight, out, bias):
            return out
        if bias is None and self._lt_takes(x.shape[0], weight) and self.lt_linear(x, weight, out):
            return out
        if bias is not None:
            torch.addmm(bias, x, weight.t(), out=out)
        else:
            torch.mm(x, weight.t(), out=out)
        return out

    @_timed("linear_gate_up_act", _weight_bytes)
    def linear_act_mul(self, x, weight, out, gate_up, act: int = 0):
        """out[T, I] = act(x @ Wg.T) * (x @ Wu.T) for weight = [Wg; Wu] ([2 I, K]).  Few bfloat16 rows: one
        kernel, the activation in the product's epilogue (gate and up never leave the chip).  Otherwise the
        product into `gate_up` [T, 2 I] and the activation kernel."""
        _need(x, "x")
        _need(out, "out")
        if self._own_linear(x, weight, out, None, act):
            return out
        # many rows: the persistent tcgen05 product with the activation in its epilogue against the library's
        # product followed by the activation kernel (measured at Qwen3-8B sizes): 300 against 310 us at 2,048 rows
        # with the library's own first algorithm, but 300 against 251 + 31 us with the library's timed choice
        # (`lt_linear`); 576 against 500 - 535 + 62 us at 4,096 rows, from where it is taken
        if x.shape[0] >= self.fused_mlp_rows and self.large_linear(x, weight, out, None, act):
            return out
        self.linear(x, weight, gate_up)
        self.act_mul(gate_up, out, act)
        return out

    @_timed("linear_head", _weight_bytes)
    def linear_f32_out(self, x, weight, out):
        """out (float32) = x @ weight.T for x/weight in float32 or bfloat16."""
        _need(out, "out", torch.float32)
        if x.dtype == torch.float32:
            torch.mm(x, weight.t(), out=out)
            return out
        if self._own_linear(x, weight, out):
            return out
        if self._lt_takes(x.shape[0], weight) and self.lt_linear(x, weight, out):
            return out
        if self._f32_out_mm is None:
            try:
                torch.mm(x[:1], weight[:8].t(), out_dtype=torch.float32)
                self._f32_out_mm = True
            except (TypeError, RuntimeError):
                self._f32_out_mm = False
        if self._f32_out_mm:
            torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
        else:
            tmp = torch.mm(x, weight.t())
            self._check(self.lib.ullm_cast_bf16_f32(_ptr(tmp), _ptr(out), tmp.numel(), _stream()), "cast")
        return out

    # -- hand-written kernels ----------------------------------------------------
    @_timed("embedding")
    def embedding(self, ids, table, out, last_tokens=None, token_req=None, req_slots=None):
        """out[t] = table[ids[t]].  With `last_tokens` (and the batch row of each token and the request
        slot of each batch row), an id of -1 means the token that request sampled last."""
        _need(ids, "ids", torch.int32)
        _need(table, "table")
        _need(out, "out", table.dtype)
        T, H = out.shape
        if ids.numel() < T or table.shape[1] != H:
            raise KernelError(f"embedding: ids {tuple(ids.shape)}, table {tuple(table.shape)}, out {tuple(out.shape)}")
        if last_tokens is not None:
            for t_, n_ in ((last_tokens, "last_tokens"), (token_req, "token_req"), (req_slots, "req_slots")):
                _need(t_, n_, torch.int32)
        self._check(self.lib.ullm_embedding(_DT[table.dtype], _ptr(ids), _ptr(table), _ptr(out), T, H,
                                            table.shape[0], _ptr(last_tokens), _ptr(token_req), _ptr(req_slots),
                                            _ptr(self.status), _stream()), "embedding")

    @_timed("gather_rows")
    def gather_rows(self, src, rows, out):
        _need(src, "src")
        _need(rows, "rows", torch.int32)
        _need(out, "out", src.dtype)
        R, C = out.shape
        if src.shape[1] != C or rows.numel() < R:
            raise KernelError(f"gather_rows: src {tuple(src.shape)}, rows {tuple(rows.shape)}, out {tuple(out.shape)}")
        self._check(self.lib.ullm_gather_rows(_DT[src.dtype], _ptr(rows), _ptr(src), _ptr(out), R, C, src.shape[0],
                                              _ptr(self.status), _stream()), "gather_rows")

    @_timed("add_rmsnorm")
    def add_rmsnorm(self, x, residual, weight, eps, out):
        _need(x, "x")
        _need(weight, "weight", torch.float32)
        _need(out, "out", x.dtype)
        if residual is not None:
            _need(residual, "residual", x.dtype)
            if residual.shape != x.shape:
                raise KernelError("add_rmsnorm: residual shape differs from x")
        rows, cols = x.shape
        if weight.numel() != cols or out.shape != x.shape:
            raise KernelError(f"add_rmsnorm: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
        self._check(self.lib.ullm_add_rmsnorm(_DT[x.dtype], _ptr(x), _ptr(residual), _ptr(weight), _ptr(out), rows,
                                              cols, float(eps), _stream()), f"add_rmsnorm (row length {cols})")

    @_timed("act_mul")
    def act_mul(self, gate_up, out, act: int = 0):
        _need(gate_up, "gate_up")
        _need(out, "out", gate_up.dtype)
        rows, inter = out.shape
        if gate_up.shape != (rows, 2 * inter):
            raise KernelError(f"act_mul: gate_up {tuple(gate_up.shape)}, out {tuple(out.shape)}")
        self._check(self.lib.ullm_act_mul(_DT[gate_up.dtype], act, _ptr(gate_up), _ptr(out), rows, inter, _stream()),
                    "act_mul")

    # -- a residual stream kept in 32-bit ---------------------------------------
    @_timed("embedding")
    def embed_scaled(self, ids, table, stream, copy=None, scale: float = 1.0, inv_freq=None, positions=None,
                     last_tokens=None, token_req=None, req_slots=None):
        """stream[t] (float32) = table[ids[t]] * scale, plus the sinusoid of positions[t] when `inv_freq`
        (float32 [ceil(hidden / 2)]) is given; `copy` (the table's dtype, optional) gets the rounded stream.
        An id of -1 is the request's last sampled token, as in `embedding`."""
        _need(ids, "ids", torch.int32)
        _need(table, "table")
        _need(stream, "stream", torch.float32)
        T, H = stream.shape
        if ids.numel() < T or table.shape[1] != H:
            raise KernelError(f"embed_scaled: ids {tuple(ids.shape)}, table {tuple(table.shape)}, stream {tuple(stream.shape)}")
        if copy is not None:
            _need(copy, "copy", table.dtype)
            if copy.shape != stream.shape:
                raise KernelError("embed_scaled: the copy's shape differs from the stream's")
        if inv_freq is not None:
            _need(inv_freq, "inv_freq", torch.float32)
            _need(positions, "positions", torch.int32)
            if inv_freq.numel() < (H + 1) // 2 or positions.numel() < T:
                raise KernelError("embed_scaled: the frequency table or the positions are too short")
        if last_tokens is not None:
            for t_, n_ in ((last_tokens, "last_tokens"), (token_req, "token_req"), (req_slots, "req_slots")):
                _need(t_, n_, torch.int32)
        self._check(self.lib.ullm_embed_scaled(_DT[table.dtype], _ptr(ids), _ptr(table), _ptr(stream), _ptr(copy), T, H,
                                               table.shape[0], float(scale), _ptr(inv_freq), _ptr(positions),
                                               _ptr(last_tokens), _ptr(token_req), _ptr(req_slots), _ptr(self.status),
                                               _stream()), "embed_scaled")

    @_timed("add_rmsnorm")
    def norm_scale_add(self, a, stream, weight, eps: float, mult: float, copy=None, next_norm=None):
        """stream (float32, in place) += mult * weight * a / sqrt(mean(a^2) + eps); `copy` (a's dtype, optional)
        gets the rounded stream.  `next_norm` = (weight2, eps2, out): the same kernel also leaves the RMSNorm of
        the updated stream in `out` (a's dtype); False is returned when it does not take the row length (nothing
        has run then)."""
        _need(a, "a")
        _need(stream, "stream", torch.float32)
        _need(weight, "weight", torch.float32)
        rows, cols = a.shape
        if stream.shape != a.shape or weight.numel() != cols:
            raise KernelError(f"norm_scale_add: a {tuple(a.shape)}, stream {tuple(stream.shape)}, weight {tuple(weight.shape)}")
        if next_norm is not None:
            w2, eps2, out = next_norm
            if copy is not None or cols * 4 > 40 * 1024:
                return False
            _need(w2, "next norm weight", torch.float32)
            _need(out, "out", a.dtype)
            if out.shape != a.shape or w2.numel() != cols:
                raise KernelError("norm_scale_add: the next norm's shapes differ")
            self._check(self.lib.ullm_norm_scale_add_norm(_DT[a.dtype], _ptr(a), _ptr(stream), _ptr(weight), rows, cols,
                                                          float(eps), float(mult), _ptr(w2), float(eps2), _ptr(out),
                                                          _stream()), "norm_scale_add_norm")
            return True
        if copy is not None:
            _need(copy, "copy", a.dtype)
            if copy.shape != a.shape:
                raise KernelError("norm_scale_add: the copy's shape differs")
        self._check(self.lib.ullm_norm_scale_add(_DT[a.dtype], _ptr(a), _ptr(stream), _ptr(weight), _ptr(copy), rows, cols,
                                                 float(eps), float(mult), _stream()), "norm_scale_add")

    @_timed("add_rmsnorm")
    def rmsnorm_rows_f32(self, stream, rows, weight, eps: float, out):
        """out[r] = weight * s / sqrt(mean(s^2) + eps) for s = stream[rows[r]] (float32 stream, `rows` int32 or
        None for all rows in order), rounded to out's dtype."""
        _need(stream, "stream", torch.float32)
        _need(weight, "weight", torch.float32)
        _need(out, "out")
        R, C = out.shape
        if stream.shape[1] != C or weight.numel() != C or (rows is None and stream.shape[0] < R):
            raise KernelError(f"rmsnorm_rows_f32: stream {tuple(stream.shape)}, out {tuple(out.shape)}")
        if rows is not None:
            _need(rows, "rows", torch.int32)
            if rows.numel() < R:
                raise KernelError("rmsnorm_rows_f32: fewer row indices than output rows")
        self._check(self.lib.ullm_rmsnorm_rows_f32(_DT[out.dtype], _ptr(stream), _ptr(rows), _ptr(weight), _ptr(out), R, C,
                                                   stream.shape[0], float(eps), _ptr(self.status), _stream()),
                    "rmsnorm_rows_f32")

    @_timed("add_rmsnorm")
    def cast_rows_f32(self, src, out):
        _need(src, "src", torch.float32)
        _need(out, "out")
        if src.shape != out.shape:
            raise KernelError("cast_rows_f32: shapes differ")
        self._check(self.lib.ullm_cast_rows_f32(_DT[out.dtype], _ptr(src), _ptr(out), src.numel(), _stream()), "cast_rows_f32")

    @_timed("act_mul")
    def act_mul_clamped(self, gate_up, out, limit: float, alpha: float):
        """out = g' * sigmoid(alpha g') * (u' + 1) with g' = min(gate, limit), u' = clamp(up, -limit, limit)."""
        _need(gate_up, "gate_up")
        _need(out, "out", gate_up.dtype)
        rows, inter = out.shape
        if gate_up.shape != (rows, 2 * inter):
            raise KernelError(f"act_mul_clamped: gate_up {tuple(gate_up.shape)}, out {tuple(out.shape)}")
        self._check(self.lib.ullm_act_mul_clamped(_DT[gate_up.dtype], _ptr(gate_up), _ptr(out), rows, inter, float(limit),
                                                  float(alpha), _stream()), "act_mul_clamped")

    # -- norms on both sides of a sub-layer, on a 32-bit stream -------------------
    @_timed("add_rmsnorm")
    def norm_add_norm(self, stream, a=None, weight=None, eps: float = 0.0, mult: float = 1.0, center: bool = False,
                      extra_rows=None, extra_vec=None, next_norm=None, plain: bool = False):
        """stream (float32, in place) += mult * weight * n(a), then += extra_rows, then += extra_vec (each part
        optional); `next_norm` = (weight2, eps2, center2, out): out = weight2 * n2(stream) rounded to out's dtype.
        n(v) = v / sqrt(mean(v^2) + eps), with `center` (v - mean) / sqrt(mean((v - mean)^2) + eps); with `plain`
        n(v) = v (a is only scaled channel by channel; `weight` None: not even that)."""
        _need(stream, "stream", torch.float32)
        rows, cols = stream.shape
        if a is not None:
            _need(a, "a")
            if weight is not None or not plain:
                _need(weight, "weight", torch.float32)
            if a.shape != stream.shape or (weight is not None and weight.numel() != cols):
                raise KernelError(f"norm_add_norm: a {tuple(a.shape)}, stream {tuple(stream.shape)}")
        if extra_rows is not None:
            _need(extra_rows, "extra_rows", torch.float32)
            if extra_rows.shape != stream.shape:
                raise KernelError("norm_add_norm: the added rows' shape differs from the stream's")
        if extra_vec is not None:
            _need(extra_vec, "extra_vec", torch.float32)
            if extra_vec.numel() != cols:
                raise KernelError("norm_add_norm: the added vector's length differs from the stream's width")
        w2 = out = None
        eps2, center2 = 0.0, False
        if next_norm is not None:
            w2, eps2, center2, out = next_norm
            _need(w2, "next norm weight", torch.float32)
            _need(out, "out")
            if out.shape != stream.shape or w2.numel() != cols:
                raise KernelError("norm_add_norm: the next norm's shapes differ")
        self._check(self.lib.ullm_norm_add_norm(
            _DT[a.dtype] if a is not None else 0, _ptr(a), _ptr(stream), _ptr(weight), rows, cols, float(eps), float(mult),
            2 if plain else int(bool(center)), _ptr(extra_rows), _ptr(extra_vec), _ptr(w2), float(eps2), int(bool(center2)),
            _DT[out.dtype] if out is not None else 0, _ptr(out), _stream()), f"norm_add_norm (row length {cols})")

    @_timed("add_rmsnorm")
    def norm_rows(self, stream, rows, weight, eps: float, out, center: bool = False):
        """out[r] = weight * n(stream[rows[r]]) (float32 stream; `rows` int32, or None for all rows in order),
        rounded to out's dtype; n as in `norm_add_norm`."""
        _need(stream, "stream", torch.float32)
        _need(weight, "weight", torch.float32)
        _need(out, "out")
        R, C = out.shape
        if stream.shape[1] != C or weight.numel() != C or (rows is None and stream.shape[0] < R):
            raise KernelError(f"norm_rows: stream {tuple(stream.shape)}, out {tuple(out.shape)}")
        if rows is not None:
            _need(rows, "rows", torch.int32)
            if rows.numel() < R:
                raise KernelError("norm_rows: fewer row indices than output rows")
        self._check(self.lib.ullm_norm_rows(_DT[out.dtype], _ptr(stream), _ptr(rows), _ptr(weight), _ptr(out), R, C,
                                            stream.shape[0], float(eps), int(bool(center)), _ptr(self.status),
                                            _stream()), f"norm_rows (row length {C})")

    @_timed("act_mul")
    def xielu(self, x, pq, out):
        """out = softplus(p) z^2 + z / 2 for z > 0, (1/2 + softplus(q)) (e^z - 1 - z) + z / 2 otherwise, with
        (p, q) = `pq` (float32 [2] on the device)."""
        _need(x, "x")
        _need(out, "out", x.dtype)
        _need(pq, "pq", torch.float32)
        if out.shape != x.shape or pq.numel() != 2:
            raise KernelError(f"xielu: x {tuple(x.shape)}, out {tuple(out.shape)}, pq {tuple(pq.shape)}")
        self._check(self.lib.ullm_xielu(_DT[x.dtype], _ptr(x), _ptr(out), x.numel(), _ptr(pq), _stream()), "xielu")

    # -- attention whose values are its keys; pooled blocks; latent attention ------
    @_timed("qk_norm_rope_store")
    def kv_shared_prepare(self, qk, q_size: int, kv_size: int, q_w, k_w, eps: float, slot_mapping, k_pages, v_pages):
        """qk [T, >= q_size + kv_size] holds q | k as projected.  With weights: q <- RMSnorm over all its q_size
        columns (in place), the likewise normed k goes to the key pages and k as projected to the value pages.
        Without: k goes to the key pages (and to `v_pages` if given)."""
        _need(qk, "qk", contiguous=False)
        _need(k_pages, "k_pages", qk.dtype)
        if qk.stride(1) != 1 or qk.shape[1] < q_size + kv_size:
            raise KernelError(f"kv_shared_prepare: qk {tuple(qk.shape)} for {q_size} + {kv_size} columns")
        if (q_w is None) != (k_w is None):
            raise KernelError("kv_shared_prepare: the norm weights of q and k come together")
        if q_w is not None:
            _need(q_w, "q_w", torch.float32)
            _need(k_w, "k_w", torch.float32)
            if q_w.numel() != q_size or k_w.numel() != kv_size:
                raise KernelError("kv_shared_prepare: the norm weights do not fit the projections")
        if v_pages is not None:
            _need(v_pages, "v_pages", qk.dtype)
            if v_pages.numel() != k_pages.numel():
                raise KernelError("kv_shared_prepare: value pages of another size than the key pages")
        if slot_mapping is not None:
            _need(slot_mapping, "slot_mapping", torch.int32)
        self._check(self.lib.ullm_kv_shared_prepare(
            _DT[qk.dtype], _ptr(qk), qk.stride(0), qk.shape[0], q_size, kv_size, _ptr(q_w), _ptr(k_w), float(eps),
            _ptr(slot_mapping), _ptr(k_pages), _ptr(v_pages), k_pages.numel() // kv_size, _ptr(self.status), _stream()),
            "kv_shared_prepare")

    @_timed("qk_norm_rope_store")
    def pool_blocks(self, positions, token_req, req_slots, block_table, page_size: int, k_pages, v_pages, pool_slots,
                    pk_pages, pv_pages, pool: int):
        """For every token whose `pool_slots` entry is not -1 (it completes a block of `pool` positions): the mean
        of the block's key rows (and value rows, when the values have pages of their own) as the pages hold them,
        written to that slot of the pooled pages."""
        for t, n in ((positions, "positions"), (token_req, "token_req"), (req_slots, "req_slots"),
                     (block_table, "block_table"), (pool_slots, "pool_slots")):
            _need(t, n, torch.int32)
        _need(k_pages, "k_pages")
        _need(pk_pages, "pk_pages", k_pages.dtype)
        row = k_pages.shape[-2] * k_pages.shape[-1]
        v_row = 0
        if (v_pages is None) != (pv_pages is None):
            raise KernelError("pool_blocks: value pages and pooled value pages come together")
        if v_pages is not None:
            _need(v_pages, "v_pages", k_pages.dtype)
            _need(pv_pages, "pv_pages", k_pages.dtype)
            v_row = v_pages.shape[-2] * v_pages.shape[-1]
        T = pool_slots.numel()
        self._check(self.lib.ullm_pool_blocks(
            _DT[k_pages.dtype], _ptr(positions), _ptr(token_req), _ptr(req_slots), _ptr(block_table), block_table.shape[1],
            page_size, k_pages.numel() // (page_size * row), _ptr(k_pages), _ptr(v_pages), row, v_row, _ptr(pool_slots),
            pk_pages.numel() // row, _ptr(pk_pages), _ptr(pv_pages), int(pool), T, _ptr(self.status), _stream()),
            "pool_blocks")

    @_timed("qk_norm_rope_store")
    def latent_prepare(self, q_full, q_lat, dkv, q_out, heads: int, dim: int, rot: int, rank: int, rot_dims: int, c_w,
                       eps: float, inv_freq, positions, slot_mapping, k_pages, interleaved: bool = True):
        """Latent attention, absorbed form.  q_full [T, heads x (dim + rot)], q_lat [heads, T, rank] (each head's
        unrotated query times its key up-projection; None: the product wrote it into q_out itself), dkv
        [T, rank + rot]; q_full and dkv may be column ranges of wider rows.  Leaves q_out [T, heads x (rank + rot)]
        = [q_lat | rotated q_rot] per head and the key row [RMSnorm(dkv[:rank]) x c_w | rotated dkv[rank:]] in
        `k_pages` at the tokens' slots.  Neighbouring dimensions (2i, 2i + 1) below `rot_dims` are rotated, or
        without `interleaved` the dimensions (i, i + rot_dims / 2)."""
        T = dkv.shape[0]
        for t, n in ((q_full, "q_full"), (dkv, "dkv")):
            _need(t, n, dkv.dtype, contiguous=False)
            if t.stride(1) != 1:
                raise KernelError(f"latent_prepare: {n} needs unit stride inside its rows")
        for t, n in ((q_out, "q_out"), (k_pages, "k_pages")) + (((q_lat, "q_lat"),) if q_lat is not None else ()):
            _need(t, n, dkv.dtype)
        _need(c_w, "c_w", torch.float32)
        _need(positions, "positions", torch.int32)
        if (q_full.shape != (T, heads * (dim + rot)) or (q_lat is not None and q_lat.shape != (heads, T, rank))
                or dkv.shape[1] != rank + rot or q_out.shape != (T, heads * (rank + rot)) or c_w.numel() != rank
                or k_pages.shape[-1] != rank + rot):
            raise KernelError("latent_prepare: shapes do not fit the sizes")
        if rot_dims:
            _need(inv_freq, "inv_freq", torch.float32)
            if inv_freq.numel() < rot_dims // 2:
                raise KernelError("latent_prepare: the frequency table is too short")
        if slot_mapping is not None:
            _need(slot_mapping, "slot_mapping", torch.int32)
        self._check(self.lib.ullm_latent_prepare(
            _DT[dkv.dtype], _ptr(q_full), _ptr(q_lat), _ptr(dkv), _ptr(q_out), T, heads, dim, rot, rank, rot_dims,
            _ptr(c_w), float(eps), _ptr(inv_freq), _ptr(positions), _ptr(slot_mapping), _ptr(k_pages),
            k_pages.numel() // (rank + rot), _ptr(self.status), _stream(), int(bool(interleaved)), q_full.stride(0),
            dkv.stride(0)), "latent_prepare")

    @_timed("qk_norm_rope_store")
    def qkv_rows_prepare(self, qkv, q_out, num_q: int, num_kv: int, head_dim: int, v_dim: int, positions, slot_mapping,
                         k_pages, v_pages, *, q_w=None, k_w=None, eps: float = 0.0, inv_freq=None, rotary_dim: int = 0,
                         interleaved: bool = False, q_head_scale=None, value_unit_norm: bool = False):
        """qkv [T, q | k | v] as projected.  q and k pass an RMS norm over the WHOLE projection (weights `q_w`
        [num_q * head_dim], `k_w` [num_kv * head_dim]; None: no norm), then the first `rotary_dim` dimensions of every
        head turn (neighbours with `interleaved`, else halves) by computed angles; q is multiplied head by head by
        `q_head_scale` [num_q] and goes to `q_out`, k to the key pages; v, with `value_unit_norm` every head divided by
        its root mean square (eps, no weight), to the value pages."""
        _need(qkv, "qkv", contiguous=False)
        _need(q_out, "q_out", qkv.dtype)
        T = qkv.shape[0]
        W = num_q * head_dim + num_kv * (head_dim + v_dim)
        if qkv.stride(1) != 1 or qkv.shape[1] < W or q_out.shape != (T, num_q * head_dim):
            raise KernelError(f"qkv_rows_prepare: qkv {tuple(qkv.shape)}, q_out {tuple(q_out.shape)}")
        if (q_w is None) != (k_w is None):
            raise KernelError("qkv_rows_prepare: the norm weights of q and k come together")
        for t_, n_, want in ((q_w, "q norm weight", num_q * head_dim), (k_w, "k norm weight", num_kv * head_dim),
                             (q_head_scale, "head factors", num_q), (inv_freq, "inv_freq", rotary_dim // 2)):
            if t_ is not None:
                _need(t_, n_, torch.float32)
                if t_.numel() < want:
                    raise KernelError(f"qkv_rows_prepare: {n_} holds {t_.numel()} values, {want} are needed")
        if rotary_dim > 0:
            if inv_freq is None:
                raise KernelError("qkv_rows_prepare: a rotation needs its frequency table")
            _need(positions, "positions", torch.int32)
        num_slots = 0
        if slot_mapping is not None:
            _need(slot_mapping, "slot_mapping", torch.int32)
            _need(k_pages, "k_pages", qkv.dtype)
            _need(v_pages, "v_pages", qkv.dtype)
            if k_pages.shape[-2:] != (num_kv, head_dim) or v_pages.shape[-2:] != (num_kv, v_dim):
                raise KernelError(f"qkv_rows_prepare: pages {tuple(k_pages.shape)} / {tuple(v_pages.shape)}")
            num_slots = k_pages.numel() // (num_kv * head_dim)
        self._check(self.lib.ullm_qkv_rows_prepare(
            _DT[qkv.dtype], _ptr(qkv), qkv.stride(0), _ptr(q_out), T, num_q, num_kv, head_dim, v_dim, _ptr(q_w), _ptr(k_w),
            float(eps), _ptr(inv_freq), int(rotary_dim), int(bool(interleaved)), _ptr(positions), _ptr(q_head_scale),
            int(bool(value_unit_norm)), _ptr(slot_mapping), _ptr(k_pages), _ptr(v_pages), num_slots, _ptr(self.status),
            _stream()), f"qkv_rows_prepare (head_dim {head_dim})")

    @_timed("add_rmsnorm")
    def concat_rows_f32(self, a, b, out):
        """out[t] = [a[t] | b[t]] rounded to out's dtype; a, b float32."""
        _need(a, "a", torch.float32)
        _need(b, "b", torch.float32)
        _need(out, "out")
        T = a.shape[0]
        if b.shape[0] != T or out.shape != (T, a.shape[1] + b.shape[1]):
            raise KernelError(f"concat_rows_f32: a {tuple(a.shape)}, b {tuple(b.shape)}, out {tuple(out.shape)}")
        self._check(self.lib.ullm_concat_rows_f32(_DT[out.dtype], _ptr(a), _ptr(b), _ptr(out), T, a.shape[1], b.shape[1],
                                                  _stream()), "concat_rows_f32")

    @_timed("act_mul")
    def sigmoid_gate(self, a, g):
        """a (in place) *= sigmoid(g), element by element; g [T, cols] may be a column range of wider rows."""
        _need(a, "a")
        _need(g, "g", a.dtype, contiguous=False)
        if g.shape != a.shape or g.stride(1) != 1:
            raise KernelError(f"sigmoid_gate: a {tuple(a.shape)}, g {tuple(g.shape)}")
        self._check(self.lib.ullm_sigmoid_gate(_DT[a.dtype], _ptr(a), _ptr(g), g.stride(0), a.shape[0], a.shape[1],
                                               _stream()), "sigmoid_gate")

    @_timed("attention")
    def windowed_attention(self, q, out, k_pages, v_pages, block_table, req_slots, cu_q, kv_len, token_req, num_q: int,
                           num_kv: int, head_dim: int, v_dim: int, page_size: int, window: int, scale: float, *,
                           slopes=None, pool: int = 0, pooled=None, gate=None, out_scale: float = 1.0,
                           num_requests: int | None = None, workspace=None):
        """Windowed attention with its further options: in bfloat16, at sizes `ullm_window_attention_supported`
        takes and with `num_requests` (the batch rows that `cu_q` describes) given, the tensor-core kernel of
        csrc/attention_window.cu; otherwise (32-bit storage, other sizes) the general kernel.  With a `workspace`
        a step of few rows cuts every row's keys into runs that run side by side (`_window_splits`).  `v_pages` None: a head's values are the first
        `v_dim` elements of its key rows.  `slopes` (float32 [num_q]): score(i, j) -= slopes[h] (i - j).  `pool` P
        with `pooled` = (pooled key pages, pooled value pages or None, their block table): blocks of P positions
        that lie wholly before the window are seen through one mean key / value each.  `gate` [T, num_q x v_dim]
        (row stride free): out *= sigmoid(gate).  `out` [T, num_q x v_dim] may be a column range of wider rows."""
        _need(q, "q", contiguous=False)
        _need(out, "out", q.dtype, contiguous=False)
        _need(k_pages, "k_pages", q.dtype)
        for t, n in ((block_table, "block_table"), (req_slots, "req_slots"), (cu_q, "cu_q"), (kv_len, "kv_len"),
                     (token_req, "token_req")):
            _need(t, n, torch.int32)
        T = out.shape[0]
        if q.stride(1) != 1 or out.stride(1) != 1 or out.shape[1] != num_q * v_dim or q.shape[1] < num_q * head_dim:
            raise KernelError(f"windowed_attention: q {tuple(q.shape)}, out {tuple(out.shape)}")
        if k_pages.shape[-3:] != (page_size, num_kv, head_dim):
            raise KernelError(f"windowed_attention: key pages {tuple(k_pages.shape)}")
        if v_pages is not None:
            _need(v_pages, "v_pages", q.dtype)
            if v_pages.shape[-3:] != (page_size, num_kv, v_dim):
                raise KernelError(f"windowed_attention: value pages {tuple(v_pages.shape)}")
        elif v_dim > head_dim:
            raise KernelError("windowed_attention: values inside the key rows cannot be wider than the keys")
        if slopes is not None:
            _need(slopes, "slopes", torch.float32)
            if slopes.numel() != num_q:
                raise KernelError("windowed_attention: one slope per head")
        pk = pv = pbt = None
        if pool:
            pk, pv, pbt = pooled
            _need(pk, "pooled key pages", q.dtype)
            _need(pbt, "pooled block table", torch.int32)
            if pk.shape[-3:] != (page_size, num_kv, head_dim) or (pv is None) != (v_pages is None):
                raise KernelError("windowed_attention: the pooled pages do not fit the pages")
            if pv is not None:
                _need(pv, "pooled value pages", q.dtype)
        if gate is not None:
            _need(gate, "gate", q.dtype, contiguous=False)
            if gate.stride(1) != 1 or gate.shape != (T, num_q * v_dim):
                raise KernelError(f"windowed_attention: gate {tuple(gate.shape)}")
        num_pages = k_pages.numel() // (page_size * num_kv * head_dim)
        p_pages = pk.numel() // (page_size * num_kv * head_dim) if pk is not None else 0
        if (self.window_attention_tc and q.dtype == torch.bfloat16 and num_requests and q.stride(0) % 8 == 0
                and out.stride(0) % 2 == 0 and out.data_ptr() % 4 == 0 and q.data_ptr() % 16 == 0
                and self.lib.ullm_window_attention_supported(head_dim, v_dim, num_q, num_kv, int(v_pages is None))):
            self.attention_path = "window_mma"
            splits = self._window_splits(T, int(num_requests), num_q, num_kv, int(window)) if workspace is not None else 1
            parts = None
            if splits > 1:
                # (rows x splits <= 64 x blocks x splits < 64 x 2.5 x SMs whenever `_window_splits` splits)
                parts = workspace.get("attn.window_parts", T * num_q * splits, v_dim + 2, torch.float32,
                                      reserve=64 * 3 * self.sm_count)
            self._check(self.lib.ullm_window_attention(
                _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                block_table.shape[1], _ptr(req_slots), _ptr(cu_q), _ptr(kv_len), T, int(num_requests), num_q, num_kv,
                head_dim, v_dim, page_size, int(window), float(scale), num_pages, _ptr(self.status), _stream(),
                _ptr(slopes), int(pool), _ptr(pk), _ptr(pv), _ptr(pbt), pbt.shape[1] if pbt is not None else 0, p_pages,
                _ptr(gate), gate.stride(0) if gate is not None else 0, float(out_scale), splits, _ptr(parts)),
                f"window_attention (key rows {head_dim}, values {v_dim}, pool {pool})")
            return
        self.attention_path = "generic"
        self._check(self.lib.ullm_paged_attention_generic_ex3(
            _DT[q.dtype], _ptr(q), q.stride(0), _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
            block_table.shape[1], _ptr(req_slots), _ptr(cu_q), _ptr(kv_len), _ptr(token_req), T, num_q, num_kv, head_dim,
            page_size, int(window), float(scale), k_pages.numel() // (page_size * num_kv * head_dim), _ptr(self.status),
            _stream(), v_dim, 0, 0.0, _ptr(slopes), int(v_pages is None), int(pool), _ptr(pk), _ptr(pv), _ptr(pbt),
            pbt.shape[1] if pbt is not None else 0,
            pk.numel() // (page_size * num_kv * head_dim) if pk is not None else 0, _ptr(gate),
            gate.stride(0) if gate is not None else 0, float(out_scale), out.stride(0)),
            f"windowed_attention (head_dim {head_dim}, values {v_dim}, pool {pool})")

    def _window_splits(self, T: int, requests: int, num_q: int, num_kv: int, window: int) -> int:
        """Into how many runs `windowed_attention` cuts a row's key tiles: one while the step's blocks (64 rows of
        a kv head each) fill half of the SMs; otherwise as many as bring two blocks per SM, at most one run per
        key tile of the window (32 without a window) and 64."""
        tokens_per_block = max(1, 64 // (num_q // num_kv))
        blocks = (max(requests, -(-T // tokens_per_block))) * num_kv
        if 2 * blocks >= self.sm_count:
            return 1
        most = -(-window // 64) + 1 if window > 0 else 32
        return max(1, min(-(-2 * self.sm_count // blocks), most, 64))

    # -- minGRU -------------------------------------------------------------------
    @_timed("mingru")
    def mingru(self, azg, a_off: int, x_off: int, g_off: int, b_z, b_x, state, cu_q, req_slots, token_req, out,
               out_scale: float, requests: int, max_q: int, fold=None):
        """azg (float32 [T, >= 3 width]): the gate's, the candidate's and the output gate's projections side by side;
        state (float32 [slots, width]) is carried; out [T, width] (any row stride) = out_scale * S_t * silu(g_t).
        `fold`: scratch for the chunked form (float32, `mingru_fold_floats`), taken for portions longer than a chunk."""
        _need(azg, "azg", torch.float32)
        _need(state, "state", torch.float32)
        _need(b_z, "b_z", torch.float32)
        _need(b_x, "b_x", torch.float32)
        _need(out, "out", contiguous=False)
        for t, n in ((cu_q, "cu_q"), (req_slots, "req_slots"), (token_req, "token_req")):
            _need(t, n, torch.int32)
        width = state.shape[1]
        if out.shape[1] != width or out.stride(1) != 1 or max(a_off, x_off, g_off) + width > azg.shape[1]:
            raise KernelError(f"mingru: azg {tuple(azg.shape)}, out {tuple(out.shape)}, width {width}")
        if fold is not None:
            _need(fold, "fold", torch.float32)
            if fold.numel() < self.mingru_fold_floats(requests, max_q, width):
                fold = None
        self._check(self.lib.ullm_mingru(
            _DT[out.dtype], _ptr(azg), azg.stride(0), a_off, x_off, g_off, _ptr(b_z), _ptr(b_x), _ptr(state),
            state.stride(0), _ptr(cu_q), _ptr(req_slots), _ptr(token_req), _ptr(out), out.stride(0), float(out_scale),
            requests, width, int(max_q), _ptr(fold), _stream()), "mingru")

    def mingru_chunk(self) -> int:
        """Portions longer than this many tokens take the chunked form when a scratch buffer is given."""
        return int(self.lib.ullm_mingru_chunk())

    def mingru_fold_floats(self, requests: int, max_q: int, width: int) -> int:
        c = self.lib.ullm_mingru_chunk()
        return 2 * requests * (-(-max_q // c)) * width

    # -- matrix memory (mLSTM) ----------------------------------------------------
    def mlstm_supported(self, heads: int, dim: int, vdim: int) -> bool:
        return bool(self.lib.ullm_mlstm_supported(heads, dim, vdim))

    def mlstm_state_floats(self, heads: int, dim: int, vdim: int) -> int:
        return int(self.lib.ullm_mlstm_state_floats(heads, dim, vdim))

    @_timed("mlstm")
    def mlstm_recurrence(self, qkv, q_off, k_off, v_off, gates, bias_i, bias_f, state, cu_q, req_slots, token_req, out,
                         requests, heads, dim, vdim, q_scale, cap):
        """The recurrence of csrc/mlstm.cu over the step's tokens, from and into the requests' state rows.
        qkv [T, *]: q, k, v at the given column offsets; gates [T, 2 heads] float32; out [T, heads * vdim] float32."""
        _need(qkv, "qkv")
        _need(gates, "gates", torch.float32)
        _need(state, "state", torch.float32)
        _need(out, "out", torch.float32)
        for t_, n_ in ((bias_i, "input gate bias"), (bias_f, "forget gate bias")):
            if t_ is not None:
                _need(t_, n_, torch.float32)
        for t_, n_ in ((cu_q, "cu_q"), (req_slots, "req_slots"), (token_req, "token_req")):
            _need(t_, n_, torch.int32)
        T = qkv.shape[0]
        if gates.shape != (T, 2 * heads) or out.shape != (T, heads * vdim) or state.dim() != 2:
            raise KernelError(f"mlstm_recurrence: qkv {tuple(qkv.shape)}, gates {tuple(gates.shape)}, out {tuple(out.shape)}")
        if max(q_off, k_off) + heads * dim > qkv.shape[1] or v_off + heads * vdim > qkv.shape[1]:
            raise KernelError("mlstm_recurrence: q, k or v lie outside the rows")
        self._check(self.lib.ullm_mlstm_recurrence(
            _DT[qkv.dtype], _ptr(qkv), qkv.stride(0), q_off, k_off, v_off, _ptr(gates), _ptr(bias_i), _ptr(bias_f),
            _ptr(state), state.stride(0), _ptr(cu_q), _ptr(req_slots), _ptr(token_req), _ptr(out), requests, heads, dim,
            vdim, float(q_scale), float(cap), state.shape[0], _ptr(self.status), _stream()),
            f"mlstm_recurrence (heads {heads}, dim {dim}, vdim {vdim})")

    @_timed("mlstm")
    def mlstm_out_gate(self, o, g, weight, eps, out, heads, vdim):
        """out = o / sqrt(mean over a head of o^2 + eps) * weight * sigmoid(g); o float32 [T, heads * vdim], g a
        view [T, heads * vdim] of the projection's rows (any row stride)."""
        _need(o, "o", torch.float32)
        _need(g, "g", out.dtype, contiguous=False)
        _need(weight, "weight", torch.float32)
        _need(out, "out")
        T = o.shape[0]
        if o.shape != (T, heads * vdim) or g.shape != o.shape or out.shape != o.shape or g.stride(1) != 1 or weight.numel() != heads * vdim:
            raise KernelError(f"mlstm_out_gate: o {tuple(o.shape)}, g {tuple(g.shape)}, out {tuple(out.shape)}")
        self._check(self.lib.ullm_mlstm_out_gate(_DT[out.dtype], _ptr(o), _ptr(g), g.stride(0), _ptr(weight), _ptr(out), T,
                                                 heads, vdim, float(eps), _stream()), "mlstm_out_gate")

    @_timed("mlstm")
    def head_norm_gate(self, o, g, weight, eps, out, heads, vdim, silu: bool = False):
        """out = o / sqrt(mean over a head of o^2 + eps) * weight * gate(g); o float32 [T, heads * vdim], g a view
        [T, heads * vdim] of the projection's rows (any row stride); weight [heads * vdim], or [vdim] shared by the
        heads; gate = sigmoid, or silu when `silu`."""
        _need(o, "o", torch.float32)
        _need(g, "g", out.dtype, contiguous=False)
        _need(weight, "weight", torch.float32)
        _need(out, "out")
        T = o.shape[0]
        if (o.shape != (T, heads * vdim) or g.shape != o.shape or out.shape != o.shape or g.stride(1) != 1
                or weight.numel() not in (vdim, heads * vdim)):
            raise KernelError(f"head_norm_gate: o {tuple(o.shape)}, g {tuple(g.shape)}, out {tuple(out.shape)}, "
                              f"weight {tuple(weight.shape)}")
        per_head = int(weight.numel() == heads * vdim and heads > 1)
        self._check(self.lib.ullm_head_norm_gate(_DT[out.dtype], _ptr(o), _ptr(g), g.stride(0), _ptr(weight), _ptr(out), T,
                                                 heads, vdim, float(eps), per_head, int(bool(silu)), _stream()),
                    "head_norm_gate")

    # -- gated linear attention ---------------------------------------------------
    def gla_supported(self, heads: int, dim: int, vdim: int) -> bool:
        return bool(self.lib.ullm_gla_supported(heads, dim, vdim))

    def gla_state_floats(self, heads: int, dim: int, vdim: int) -> int:
        return int(self.lib.ullm_gla_state_floats(heads, dim, vdim))

    @_timed("gla")
    def gla_recurrence(self, qkv, q_off, k_off, v_off, z, z_bias, inv_tau, q_scale, state, cu_q, req_slots, token_req,
                       out, requests, heads, dim, vdim):
        """The recurrence of csrc/gla.cu over the step's tokens, from and into the requests' state rows.
        qkv [T, *]: q, k, v at the given column offsets; z [T, heads * dim] float32 (the decay's projection, a view
        with any row stride; the kernel REPLACES it by the decays), `z_bias` float32 [heads * dim] or None;
        out [T, heads * vdim] float32."""
        _need(qkv, "qkv")
        _need(z, "z", torch.float32, contiguous=False)
        _need(state, "state", torch.float32)
        _need(out, "out", torch.float32)
        if z_bias is not None:
            _need(z_bias, "decay bias", torch.float32)
        for t_, n_ in ((cu_q, "cu_q"), (req_slots, "req_slots"), (token_req, "token_req")):
            _need(t_, n_, torch.int32)
        T = qkv.shape[0]
        if z.shape != (T, heads * dim) or z.stride(1) != 1 or out.shape != (T, heads * vdim) or state.dim() != 2:
            raise KernelError(f"gla_recurrence: qkv {tuple(qkv.shape)}, z {tuple(z.shape)}, out {tuple(out.shape)}")
        if max(q_off, k_off) + heads * dim > qkv.shape[1] or v_off + heads * vdim > qkv.shape[1]:
            raise KernelError("gla_recurrence: q, k or v lie outside the rows")
        if z_bias is not None and z_bias.numel() != heads * dim:
            raise KernelError("gla_recurrence: the decay bias has the wrong length")
        self._check(self.lib.ullm_gla_recurrence(
            _DT[qkv.dtype], _ptr(qkv), qkv.stride(0), q_off, k_off, v_off, _ptr(z), z.stride(0), _ptr(z_bias),
            float(inv_tau), float(q_scale), _ptr(state), state.stride(0), _ptr(cu_q), _ptr(req_slots), _ptr(token_req),
            _ptr(out), T, requests, heads, dim, vdim, state.shape[0], _ptr(self.status), _stream()),
            f"gla_recurrence (heads {heads}, dim {dim}, vdim {vdim})")

    # -- sub-layers added to a 32-bit stream through gates; a per-token side input ----------
    @_timed("add_rmsnorm")
    def gated_add_f32(self, a, f, gates, b1, b2, stream, copy=None):
        """stream (float32, in place) += sigmoid(gates[:, :W] + b1) * a (+ sigmoid(gates[:, W:] + b2) * f when f is
        given); `copy` (a's dtype, optional) gets the rounded stream.  gates float32 [T, W or 2 W]."""
        _need(a, "a")
        _need(gates, "gates", torch.float32)
        _need(stream, "stream", torch.float32)
        _need(b1, "b1", torch.float32)
        T, W = a.shape
        if stream.shape != a.shape or gates.shape != (T, W * (2 if f is not None else 1)) or b1.numel() != W:
            raise KernelError(f"gated_add_f32: a {tuple(a.shape)}, gates {tuple(gates.shape)}, stream {tuple(stream.shape)}")
        if f is not None:
            _need(f, "f", a.dtype)
            _need(b2, "b2", torch.float32)
            if f.shape != a.shape or b2.numel() != W:
                raise KernelError("gated_add_f32: the second sub-layer's shapes differ")
        if copy is not None:
            _need(copy, "copy", a.dtype)
            if copy.shape != a.shape:
                raise KernelError("gated_add_f32: the copy's shape differs")
        self._check(self.lib.ullm_gated_add_f32(_DT[a.dtype], _ptr(a), _ptr(f), _ptr(gates), gates.stride(0), _ptr(b1),
                                                _ptr(b2 if f is not None else None), _ptr(stream), _ptr(copy), T, W,
                                                _stream()), "gated_add_f32")

    @_timed("act_mul")
    def side_gate_mul(self, s, ids, table, offset: int, out, last_tokens=None, token_req=None, req_slots=None):
        """out[t] = gelu_tanh(s[t]) * table[ids[t], offset : offset + cols]; an id of -1 is the request's last
        sampled token, as in `embedding`."""
        _need(s, "s")
        _need(ids, "ids", torch.int32)
        _need(table, "table", s.dtype)
        _need(out, "out", s.dtype)
        T, C = s.shape
        if out.shape != s.shape or ids.numel() < T or table.dim() != 2 or offset < 0 or offset + C > table.shape[1]:
            raise KernelError(f"side_gate_mul: s {tuple(s.shape)}, table {tuple(table.shape)}, offset {offset}")
        if last_tokens is not None:
            for t_, n_ in ((last_tokens, "last_tokens"), (token_req, "token_req"), (req_slots, "req_slots")):
                _need(t_, n_, torch.int32)
        self._check(self.lib.ullm_side_gate_mul(_DT[s.dtype], _ptr(s), _ptr(ids), _ptr(table), table.stride(0), int(offset),
                                                _ptr(out), T, C, table.shape[0], _ptr(last_tokens), _ptr(token_req),
                                                _ptr(req_slots), _ptr(self.status), _stream()), "side_gate_mul")

    @_timed("linear_head")
    def softcap_f32(self, x, cap: float):
        """x (float32, in place) = cap * tanh(x / cap)."""
        _need(x, "x", torch.float32)
        self._check(self.lib.ullm_softcap_f32(_ptr(x), x.numel(), float(cap), _stream()), "softcap_f32")

    # -- between an attention's projection and its scores, in general form ----------------
    @_timed("qk_norm_rope_store")
    def qkv_prepare(self, qkv, q_out, num_q, num_kv, head_dim, v_dim, positions, slot_mapping, k_pages, v_pages, *,
                    conv_w=None, taps: int = 0, conv_state=None, cu_q=None, token_req=None, req_slots=None,
                    inv_freq=None, rotary_dim: int = 0, q_w=None, k_w=None, norm_first: bool = False,
                    norm_last: bool = False, eps: float = 0.0, vmix_mode: int = 0, vmix_lambda=None, v_first=None):
        """See csrc/attention_prep.cu: short convolution (with the requests' state rows), norm, rotation by computed
        angles, unit norm, value mixing, cache stores; q goes to `q_out` [T, num_q * head_dim]."""
        _need(qkv, "qkv")
        _need(q_out, "q_out", qkv.dtype)
        T, W = qkv.shape
        if W != num_q * head_dim + num_kv * (head_dim + v_dim) or q_out.shape != (T, num_q * head_dim):
            raise KernelError(f"qkv_prepare: qkv {tuple(qkv.shape)}, q_out {tuple(q_out.shape)}")
        for t_, n_ in ((token_req, "token_req"), (positions, "positions")):
            _need(t_, n_, torch.int32)
        state_stride = state_slots = 0
        if conv_w is not None:
            _need(conv_w, "conv_w", qkv.dtype)
            if conv_w.shape != (W, taps):
                raise KernelError(f"qkv_prepare: conv_w {tuple(conv_w.shape)} != ({W}, {taps})")
            for t_, n_ in ((cu_q, "cu_q"), (req_slots, "req_slots")):
                _need(t_, n_, torch.int32)
            if taps > 1:
                _need(conv_state, "conv_state", torch.float32)
                if conv_state.dim() != 2 or conv_state.shape[1] < (taps - 1) * W:
                    raise KernelError(f"qkv_prepare: conv_state {tuple(conv_state.shape)} is too small")
                state_stride, state_slots = conv_state.stride(0), conv_state.shape[0]
        for t_, n_ in ((inv_freq, "inv_freq"), (q_w, "q norm weight"), (k_w, "k norm weight"), (vmix_lambda, "vmix")):
            if t_ is not None:
                _need(t_, n_, torch.float32)
        if rotary_dim > 0 and (inv_freq is None or inv_freq.numel() < rotary_dim // 2):
            raise KernelError("qkv_prepare: the frequency table is too short")
        if v_first is not None:
            _need(v_first, "v_first", qkv.dtype)
            if v_first.shape != (T, num_kv * v_dim):
                raise KernelError(f"qkv_prepare: v_first {tuple(v_first.shape)} != ({T}, {num_kv * v_dim})")
        num_slots = 0
        if slot_mapping is not None:
            _need(slot_mapping, "slot_mapping", torch.int32)
            _need(k_pages, "k_pages", qkv.dtype)
            _need(v_pages, "v_pages", qkv.dtype)
            if k_pages.shape[-2:] != (num_kv, head_dim) or v_pages.shape[-2:] != (num_kv, v_dim):
                raise KernelError(f"qkv_prepare: pages {tuple(k_pages.shape)} / {tuple(v_pages.shape)}")
            num_slots = k_pages.numel() // (num_kv * head_dim)
        self._check(self.lib.ullm_qkv_prepare(
            _DT[qkv.dtype], _ptr(qkv), qkv.stride(0), T, num_q, num_kv, head_dim, v_dim, _ptr(conv_w), int(taps),
            _ptr(conv_state), state_stride, _ptr(cu_q), _ptr(token_req), _ptr(req_slots), state_slots, _ptr(positions),
            _ptr(inv_freq), int(rotary_dim), _ptr(q_w), _ptr(k_w), int(norm_first), int(norm_last), float(eps),
            int(vmix_mode), _ptr(vmix_lambda), _ptr(v_first), _ptr(slot_mapping), _ptr(k_pages), _ptr(v_pages), num_slots,
            _ptr(q_out), _ptr(self.status), _stream()), f"qkv_prepare (head_dim {head_dim})")

    @_timed("qk_norm_rope_store")
    def conv_state_update(self, qkv, taps: int, conv_state, cu_q, token_req, req_slots, requests: int):
        """After `qkv_prepare` of a step: the requests' state rows take the last taps - 1 projected rows."""
        _need(qkv, "qkv")
        _need(conv_state, "conv_state", torch.float32)
        for t_, n_ in ((cu_q, "cu_q"), (token_req, "token_req"), (req_slots, "req_slots")):
            _need(t_, n_, torch.int32)
        self._check(self.lib.ullm_conv_state_update(_DT[qkv.dtype], _ptr(qkv), qkv.stride(0), qkv.shape[1], int(taps),
                                                    _ptr(conv_state), conv_state.stride(0), _ptr(cu_q), _ptr(token_req),
                                                    _ptr(req_slots), conv_state.shape[0], int(requests), _stream()),
                    "conv_state_update")

    @_timed("attention")
    def mix_heads(self, parts, mix, out, num_q, num_kv, v_dim):
        """out[t, h] = sum_g mix[h, g] * parts[t, g, kv head of h] (parts float32 [T, num_q * num_kv * v_dim])."""
        _need(parts, "parts", torch.float32)
        _need(mix, "mix", torch.float32)
        _need(out, "out")
        T = out.shape[0]
        if parts.shape != (T, num_q * num_kv * v_dim) or out.shape[1] != num_q * v_dim or mix.shape != (num_q, num_q):
            raise KernelError(f"mix_heads: parts {tuple(parts.shape)}, mix {tuple(mix.shape)}, out {tuple(out.shape)}")
        self._check(self.lib.ullm_mix_heads(_DT[out.dtype], _ptr(parts), _ptr(mix), _ptr(out), T, num_q, num_kv, v_dim,
                                            _stream()), "mix_heads")

    # -- routed experts -----------------------------------------------------------
    @_timed("moe")
    def moe_route(self, logits, choice, weight, top: int, softmax_scores: bool = False, renormalize: bool = False,
                  correction=None, experts: int | None = None):
        """`experts`: the router's outputs, when the logits' rows hold further columns behind them.  `correction`
        (float32 [experts]): added to the scores for the choice; the weights stay the scores."""
        _need(logits, "router logits", torch.float32)
        _need(choice, "choice", torch.int32)
        _need(weight, "weight", torch.float32)
        T = logits.shape[0]
        E = logits.shape[1] if experts is None else int(experts)
        if choice.numel() < T * top or weight.numel() < T * top or E > logits.shape[1]:
            raise KernelError("moe_route: outputs too small")
        if correction is not None:
            _need(correction, "correction", torch.float32)
            if correction.numel() != E:
                raise KernelError(f"moe_route: {correction.numel()} corrections for {E} router outputs")
        self._check(self.lib.ullm_moe_route(_ptr(logits), logits.stride(0), _ptr(correction), _ptr(choice), _ptr(weight), T,
                                            E, top, int(softmax_scores), int(renormalize), _stream()),
                    f"moe_route ({E} experts, top {top})")

    @_timed("moe")
    def moe_arrange(self, choice, pairs: int, experts: int, offsets, sorted_pairs, place):
        for t_, n_ in ((choice, "choice"), (offsets, "offsets"), (sorted_pairs, "sorted"), (place, "place")):
            _need(t_, n_, torch.int32)
        if offsets.numel() < experts + 1 or sorted_pairs.numel() < pairs or place.numel() < pairs:
            raise KernelError("moe_arrange: outputs too small")
        self._check(self.lib.ullm_moe_arrange(_ptr(choice), pairs, experts, _ptr(offsets), _ptr(sorted_pairs), _ptr(place),
                                              _stream()), f"moe_arrange ({experts} experts)")

    @_timed("moe", lambda x, weights, *r: weights.numel() * weights.element_size())
    def moe_grouped_linear(self, x, weights, offsets, sorted_pairs, pair_weight, out, top: int, rows_from_pairs: bool,
                           gated: bool, act: int = 0, limit: float = 0.0, alpha: float = 1.0):
        """out[p] = W_e . x[row(p)] for every place p of every expert e (see csrc/moe.cu); weights
        [experts, (2 if gated) * n_out, k].  `act` 2: the clamped gate with `limit` and `alpha`."""
        _need(x, "x")
        _need(weights, "expert weights", x.dtype)
        _need(out, "out", x.dtype)
        E, N, K = weights.shape
        pairs, n_out = out.shape
        if N != (2 if gated else 1) * n_out or x.shape[1] != K:
            raise KernelError(f"moe_grouped_linear: x {tuple(x.shape)}, weights {tuple(weights.shape)}, out {tuple(out.shape)}")
        if pair_weight is not None:
            _need(pair_weight, "pair weights", torch.float32)
        self._check(self.lib.ullm_moe_grouped_linear(
            _DT[x.dtype], _ptr(x), x.stride(0), _ptr(weights), weights.stride(0), _ptr(offsets), _ptr(sorted_pairs),
            _ptr(pair_weight), _ptr(out), pairs, E, top, int(rows_from_pairs), n_out, K, int(gated), act, float(limit),
            float(alpha), _stream()),
            f"moe_grouped_linear ({E} experts, {N} x {K})")

    def moe_force_plain(self, on: bool) -> None:
        """True: the grouped product never takes its tensor-core kernel (tests compare the two)."""
        self.lib.ullm_moe_force_plain(1 if on else 0)

    @_timed("moe")
    def _combine_extras(self, what, rows, T, C, top, passing, shared):
        """Checked (choice, experts, x, x stride, shared rows, shared gate, gate stride) of the two combine calls."""
        choice = x = s_rows = s_gate = None
        experts = x_stride = g_stride = 0
        if passing is not None:
            choice, experts, x = passing
            _need(choice, "choice", torch.int32)
            _need(x, "x", rows.dtype, contiguous=False)
            if x.shape != (T, C) or x.stride(1) != 1 or choice.numel() < T * top:
                raise KernelError(f"{what}: the passing experts' input does not fit")
            x_stride = x.stride(0)
        if shared is not None:
            s_rows, s_gate = shared
            _need(s_rows, "shared rows", rows.dtype)
            if s_rows.shape != (T, C):
                raise KernelError(f"{what}: the shared expert's rows do not fit")
            if s_gate is not None:
                _need(s_gate, "shared gate", torch.float32, contiguous=False)
                if s_gate.shape[0] != T:
                    raise KernelError(f"{what}: one gate number per token")
                g_stride = s_gate.stride(0)
        return choice, int(experts), x, x_stride, s_rows, s_gate, g_stride

    @_timed("moe")
    def moe_combine(self, rows, place, pair_weight, y, top: int, passing=None, shared=None):
        """`passing` = (choice, experts, x): a choice at or beyond `experts` adds its weight times the token's row of
        x [T, cols] instead of an expert's row.  `shared` = (rows [T, cols], gate or None): added to every token,
        times sigmoid(gate[t]) (float32, one number per token, any row stride)."""
        _need(rows, "rows")
        _need(place, "place", torch.int32)
        _need(y, "y", rows.dtype)
        T, C = y.shape
        if rows.shape[1] != C or rows.shape[0] < T * top:
            raise KernelError("moe_combine: shapes differ")
        choice, experts, x, x_stride, s_rows, s_gate, g_stride = self._combine_extras("moe_combine", rows, T, C, top,
                                                                                      passing, shared)
        self._check(self.lib.ullm_moe_combine(_DT[y.dtype], _ptr(rows), _ptr(place), _ptr(pair_weight), _ptr(y), T, top, C,
                                              _ptr(choice), experts, _ptr(x), x_stride, _ptr(s_rows), _ptr(s_gate),
                                              g_stride, _stream()), "moe_combine")

    @_timed("moe")
    def moe_combine_add_norm(self, rows, place, pair_weight, top: int, stream, scale=None, next_norm=None, passing=None,
                             shared=None) -> bool:
        """stream (float32 [T, cols], in place) += scale * (the sum `moe_combine` forms), the sum kept in 32-bit;
        `scale` float32 [cols] or None.  `next_norm` = (weight2, eps2, out): out = the RMS norm of the updated rows, in
        the rows' dtype (it may be the passing experts' x).  False when the kernel does not take the row length
        (nothing has run then)."""
        _need(rows, "rows")
        _need(place, "place", torch.int32)
        _need(stream, "stream", torch.float32)
        T, C = stream.shape
        if rows.shape[1] != C or rows.shape[0] < T * top:
            raise KernelError("moe_combine_add_norm: shapes differ")
        if C * 4 > 160 * 1024:
            return False
        if scale is not None:
            _need(scale, "scale", torch.float32)
            if scale.numel() != C:
                raise KernelError("moe_combine_add_norm: the scale's length differs from the stream's width")
        w2 = out = None
        eps2 = 0.0
        if next_norm is not None:
            w2, eps2, out = next_norm
            _need(w2, "next norm weight", torch.float32)
            _need(out, "out", rows.dtype)
            if out.shape != (T, C) or w2.numel() != C:
                raise KernelError("moe_combine_add_norm: the next norm's shapes differ")
        choice, experts, x, x_stride, s_rows, s_gate, g_stride = self._combine_extras("moe_combine_add_norm", rows, T, C,
                                                                                      top, passing, shared)
        self._check(self.lib.ullm_moe_combine_add_norm(
            _DT[rows.dtype], _ptr(rows), _ptr(place), _ptr(pair_weight), T, top, C, _ptr(choice), experts, _ptr(x),
            x_stride, _ptr(s_rows), _ptr(s_gate), g_stride, _ptr(stream), _ptr(scale), _ptr(w2), float(eps2), _ptr(out),
            _stream()), "moe_combine_add_norm")
        return True

    def check_attention_sizes(self, *a):
        check_attention_sizes(*a)

    @_timed("qk_norm_rope_store")
    def qk_norm_rope_store(self, qkv, num_q, num_kv, head_dim, q_w, k_w, eps, cos, sin, rotary_dim, positions,
                           slot_mapping, k_pages, v_pages, v_dim: int | None = None, kv_in_row: bool = True):
        """`v_dim`: head size of the values when it differs from the keys'; `kv_in_row` False: the rows hold the
        query heads only (nothing is stored)."""
        _need(qkv, "qkv")
        T, W = qkv.shape
        v_dim = head_dim if v_dim is None else v_dim
        want = num_q * head_dim + ((num_kv * (head_dim + v_dim)) if kv_in_row else 0)
        if W != want:
            raise KernelError(f"qk_norm_rope_store: qkv row length {W} != {want} (Hq D + Hkv (D + Dv))")
        for t, n in ((q_w, "q_norm weight"), (k_w, "k_norm weight"), (cos, "cos table"), (sin, "sin table")):
            if t is not None:
                _need(t, n, torch.float32)
        max_pos = 0
        if rotary_dim > 0:
            if cos is None or sin is None or cos.shape != sin.shape or cos.shape[1] != rotary_dim // 2:
                raise KernelError("qk_norm_rope_store: cos/sin tables must be [positions, rotary_dim / 2]")
            max_pos = cos.shape[0]
            _need(positions, "positions", torch.int32)
        num_slots = 0
        if not kv_in_row:
            slot_mapping = None
        if slot_mapping is not None:
            _need(slot_mapping, "slot_mapping", torch.int32)
            _need(k_pages, "k_pages", qkv.dtype)
            _need(v_pages, "v_pages", qkv.dtype)
            if k_pages.shape[-2:] != (num_kv, head_dim) or v_pages.shape[-2:] != (num_kv, v_dim) \
                    or v_pages.shape[:-1] != k_pages.shape[:-1]:
                raise KernelError(f"qk_norm_rope_store: pages {tuple(k_pages.shape)} / {tuple(v_pages.shape)} do not end "
                                  f"in (Hkv, D) / (Hkv, Dv)")
            num_slots = k_pages.numel() // (num_kv * head_dim)
        if v_dim == head_dim and kv_in_row:
            code = self.lib.ullm_qk_norm_rope_store(
                _DT[qkv.dtype], _ptr(qkv), T, num_q, num_kv, head_dim, _ptr(q_w), _ptr(k_w), float(eps), _ptr(cos),
                _ptr(sin), rotary_dim, max_pos, _ptr(positions), _ptr(slot_mapping), _ptr(k_pages), _ptr(v_pages),
                num_slots, _ptr(self.status), _stream())
        else:
            code = self.lib.ullm_qk_norm_rope_store_ex(
                _DT[qkv.dtype], _ptr(qkv), T, num_q, num_kv, head_dim, _ptr(q_w), _ptr(k_w), float(eps), _ptr(cos),
                _ptr(sin), rotary_dim, max_pos, _ptr(positions), _ptr(slot_mapping), _ptr(k_pages), _ptr(v_pages),
                num_slots, _ptr(self.status), _stream(), v_dim, int(kv_in_row))
        self._check(code, f"qk_norm_rope_store (head_dim {head_dim})")

    @_timed("qk_norm_rope_store")
    def qk_norm_in_place(self, qkv, num_q, num_kv, head_dim, q_w, k_w, eps):
        """Per-head RMSNorm of the queries and the keys of `qkv` ([T, (Hq + 2 Hkv) D]) where they lie; nothing is
        stored in a cache.  (For a position encoding with code of its own, which then changes q and k.)"""
        _need(qkv, "qkv")
        T, W = qkv.shape
        if W != (num_q + 2 * num_kv) * head_dim:
            raise KernelError(f"qk_norm_in_place: qkv row length {W} != (Hq + 2 Hkv) * D")
        for t, n in ((q_w, "q_norm weight"), (k_w, "k_norm weight")):
            if t is not None:
                _need(t, n, torch.float32)
        self._check(self.lib.ullm_qk_norm_in_place(_DT[qkv.dtype], _ptr(qkv), T, num_q, num_kv, head_dim, _ptr(q_w),
                                                   _ptr(k_w), float(eps), _ptr(self.status), _stream()),
                    f"qk_norm_in_place (head_dim {head_dim})")

    def _decode_choice(self, T, ragged, num_q, num_kv, head_dim, page_size, row_stride) -> str:
        """Which decode attention kernel takes T one-token rows: "tcgen05", "balanced" or "split"."""
        balanced = ragged if self.use_balanced_decode == "auto" else self.use_balanced_decode
        if (self.use_tcgen05_decode and self.lib.ullm_decode_attention_tcgen05_supported(
                head_dim, num_q, num_kv, T, page_size) and row_stride % head_dim == 0):
            return "tcgen05"
        if balanced and self.lib.ullm_decode_attention_balanced_supported(head_dim, num_q, num_kv, T, page_size):
            return "balanced"
        return "split"

    def decode_fusion_applies(self, ctx, qkv, num_q, num_kv, head_dim, page_size, rotary_dim, cos,
                              ragged: bool = False) -> bool:
        """True when the step's attention is the per-request decode kernel and that kernel can prepare q, k and v
        itself (norm, rotation, cache write): the caller then skips `qk_norm_rope_store` and hands the pieces to
        `paged_attention(..., fuse=...)`."""
        T = qkv.shape[0]
        return bool(self.fuse_decode_rope and ctx is not None and ctx.decode_only and T == ctx.num_requests
                    and qkv.dtype == torch.bfloat16 and cos is not None and rotary_dim == head_dim
                    and self.lib.ullm_decode_attention_supported(head_dim, num_q, num_kv)
                    and self._decode_choice(T, ragged, num_q, num_kv, head_dim, page_size,
                                            qkv.stride(0)) == "split")

    def _decode_rows(self, qkv, out, k_pages, v_pages, block_table, req_slots, kv_len, num_q, num_kv, head_dim,
                     page_size, window, scale, num_pages, ragged, ctx, fuse=None, keep_first: int = 0,
                     softcap: float = 0.0, parts=None) -> None:
        """Decode attention of T one-token rows (row i belongs to request row i): streams the pages once.
        `keep_first` > 0 (with a window), `softcap` > 0 (capped scores) or `parts` (every head's weights on every
        kv head's values, 32-bit [T, num_q * num_kv * head_dim]; `out` unused): the per-request split kernel, the
        one that takes them."""
        T = qkv.shape[0]
        choice = self._decode_choice(T, ragged, num_q, num_kv, head_dim, page_size, qkv.stride(0))
        if keep_first > 0 or softcap > 0 or parts is not None:
            choice = "split"
        if fuse is not None and choice != "split":
            raise KernelError("decode attention: q and k were left unprepared for a kernel that does not prepare them")
        tc = choice == "tcgen05"
        if choice != "split":
            # both kernels cut the batch's keys evenly (over blocks, over warps) and share the scratch arrays
            # and the merge kernel for the pairs that a cut went through
            key = (head_dim, num_q, num_kv)
            if key not in self._decb:
                n = self.lib.ullm_decode_attention_balanced_scratch_floats(head_dim, num_q // num_kv)
                if head_dim == 128:
                    n = max(n, self.lib.ullm_decode_attention_tcgen05_scratch_floats(num_q // num_kv))
                if n <= 0:
                    raise KernelError("decode attention: cannot size its grid on this device")
                self._decb[key] = (torch.empty(n, dtype=torch.float32, device="cuda"),
                                   torch.zeros(513, dtype=torch.int32, device="cuda"),
                                   torch.zeros(512 * num_q, dtype=torch.int32, device="cuda"))
            part, prefix, flags = self._decb[key]
            fn = self.lib.ullm_decode_attention_tcgen05 if tc else self.lib.ullm_decode_attention_balanced
            self._check(fn(
                _ptr(qkv), qkv.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                _ptr(req_slots), _ptr(kv_len), _ptr(out), _ptr(part), _ptr(prefix), _ptr(flags), T, num_q, num_kv, head_dim,
                page_size, int(window), float(scale), num_pages, _ptr(self.status), _stream()),
                f"decode_attention_{'tcgen05' if tc else 'balanced'} (head_dim {head_dim})")
            self.launches += 1  # the merge of the shared pairs
            self.attention_path = "decode_tcgen05" if tc else "decode_balanced"
            return
        # Up to 8 rows (the steps that run under dependent launch) the splits of a request merge inside a
        # thread-block cluster: no merge kernel stands between the attention and the output projection, whose ring
        # fills meanwhile.  The cluster is the largest power of two that keeps all blocks in one wave of two per
        # SM (8 requests x 8 kv heads: 4 splits, 3.59 ms per step against 3.87 with 7 splits and the merge kernel;
        # 3, 5, 6, 7 and 8 splits: 3.70, 4.06, 3.98, 3.93, 4.06).  More rows: splits by `decode_split_target`,
        # merged by the second kernel.
        cluster = T <= max(8, self.stream_all_rows) if self.decode_cluster_merge == "auto" else self.decode_cluster_merge
        self.lib.ullm_decode_attention_cluster_merge(1 if cluster else 0)
        pairs = num_kv * (num_kv if parts is not None else 1)  # (key head, value head) pairs a request brings
        if cluster and self.decode_cluster_merge == "auto":
            splits = 8
            while splits > 1 and T * pairs * splits > 2 * self.sm_count:
                splits //= 2
        else:
            splits = max(1, min(8 if cluster else 32, -(-self.decode_split_target // (T * pairs))))
            # (request, kv head) pairs that fill half of the places on the SMs or more (two blocks per SM), but not
            # more than all of them, run unsplit: one wave, no merge launch (24 x 2,048 tokens, 8 kv heads: 46 us
            # against 50 with 3 splits and 58 with 2; 32 x 2,048: 52 against 61 with 2 splits)
            if self.decode_cluster_merge == "auto" and self.sm_count <= T * pairs <= 2 * self.sm_count:
                splits = 1
        # (splits x rows stays below the blocks aimed for, per kv head, plus one split per row)
        o_rep = num_kv if parts is not None else 1
        most = num_q * o_rep * (self.decode_split_target // pairs + max(T, getattr(ctx.workspace, "max_requests", 0)))
        scratch = ctx.workspace.get("attn.decode_scratch", T * num_q * o_rep * splits, head_dim + 2, torch.float32,
                                    reserve=most)
        if fuse is not None:
            for t, n in ((fuse["cos"], "cos table"), (fuse["sin"], "sin table")):
                _need(t, n, torch.float32)
            _need(fuse["positions"], "positions", torch.int32)
            self._check(self.lib.ullm_decode_attention_fused(
                _ptr(qkv), qkv.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                _ptr(req_slots), _ptr(kv_len), _ptr(out), _ptr(scratch), T, num_q, num_kv, head_dim, page_size,
                int(window), float(scale), splits, num_pages, _ptr(fuse["q_w"]), _ptr(fuse["k_w"]), float(fuse["eps"]),
                _ptr(fuse["cos"]), _ptr(fuse["sin"]), fuse["cos"].shape[0], _ptr(fuse["positions"]),
                _ptr(fuse["slot_mapping"]), _ptr(self.status), _stream()),
                f"decode_attention_fused (head_dim {head_dim})")
        elif parts is not None:
            self._check(self.lib.ullm_decode_attention_parts(
                _ptr(qkv), qkv.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                _ptr(req_slots), _ptr(kv_len), _ptr(parts), _ptr(scratch), T, num_q, num_kv, head_dim, page_size,
                int(window), float(scale), splits, num_pages, _ptr(self.status), _stream(), int(keep_first)),
                f"decode_attention (head_dim {head_dim}, parts)")
        elif softcap > 0:
            self._check(self.lib.ullm_decode_attention_capped(
                _ptr(qkv), qkv.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                _ptr(req_slots), _ptr(kv_len), _ptr(out), _ptr(scratch), T, num_q, num_kv, head_dim, page_size,
                int(window), float(scale), splits, num_pages, _ptr(self.status), _stream(), int(keep_first),
                float(softcap)), f"decode_attention (head_dim {head_dim}, cap {softcap})")
        elif keep_first > 0:
            self._check(self.lib.ullm_decode_attention_kept(
                _ptr(qkv), qkv.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                _ptr(req_slots), _ptr(kv_len), _ptr(out), _ptr(scratch), T, num_q, num_kv, head_dim, page_size,
                int(window), float(scale), splits, num_pages, _ptr(self.status), _stream(), int(keep_first)),
                f"decode_attention (head_dim {head_dim}, first {keep_first} kept)")
        else:
            self._check(self.lib.ullm_decode_attention(
                _ptr(qkv), qkv.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                _ptr(req_slots), _ptr(kv_len), _ptr(out), _ptr(scratch), T, num_q, num_kv, head_dim, page_size,
                int(window), float(scale), splits, num_pages, _ptr(self.status), _stream()),
                f"decode_attention (head_dim {head_dim})")
        if splits > 1 and not self.lib.ullm_decode_attention_last_used_cluster():
            self.launches += 1  # the merge of the splits
        self.attention_path = "decode"
        return

    @_timed("attention")
    def paged_attention(self, qkv, out, k_pages, v_pages, block_table, req_slots, cu_q, kv_len, token_req, num_q, num_kv,
                        head_dim, page_size, window, scale, ctx=None, fuse=None, ragged: bool = False,
                        v_dim: int | None = None, keep_first: int = 0, softcap: float = 0.0, parts=None,
                        general: bool = False):
        """Attention of every row of the flat batch over its request's pages.
        `qkv` holds q in its first num_q * head_dim columns.  `fuse` (only after `decode_fusion_applies` said
        yes): q, k and v are as the projection left them, and the kernel norms, rotates and stores them itself;
        a dict with q_w, k_w (or None), eps, cos, sin, positions, slot_mapping (or None).  `ragged` (decode
        steps): the caller found the requests' lengths very unequal, which picks the batch-balanced kernel."""
        _need(qkv, "qkv")
        _need(out, "out", qkv.dtype)
        _need(k_pages, "k_pages", qkv.dtype)
        _need(v_pages, "v_pages", qkv.dtype)
        for t, n in ((block_table, "block_table"), (req_slots, "req_slots"), (cu_q, "cu_q"), (kv_len, "kv_len"), (token_req, "token_req")):
            _need(t, n, torch.int32)
        T = out.shape[0]
        v_dim = head_dim if v_dim is None else v_dim
        if out.shape[1] != num_q * v_dim or qkv.shape[0] < T:
            raise KernelError(f"paged_attention: out {tuple(out.shape)}, qkv {tuple(qkv.shape)}")
        if k_pages.shape[-3:] != (page_size, num_kv, head_dim) or v_pages.shape[-3:] != (page_size, num_kv, v_dim):
            raise KernelError(f"paged_attention: pages {tuple(k_pages.shape)} / {tuple(v_pages.shape)} != "
                              f"[*, {page_size}, {num_kv}, {head_dim} / {v_dim}]")
        num_pages = k_pages.numel() // (page_size * num_kv * head_dim)
        if keep_first > 0 and not window:
            keep_first = 0
        if softcap > 0 or parts is not None or general:
            # capped scores, weights applied to every kv head's values (for `mix_heads`), or a caller that has
            # prepared q itself and asks for the general kernel
            if fuse is not None:
                raise KernelError("paged_attention: q and k were left unprepared, but the general kernel takes this step")
            if parts is not None:
                _need(parts, "parts", torch.float32)
                if parts.shape != (T, num_q * num_kv * v_dim):
                    raise KernelError(f"paged_attention: parts {tuple(parts.shape)}")
            # bfloat16 at head sizes 64 / 128 with values as wide as keys: the tensor-core kernels.  Decode steps
            # stream their pages through the split decode kernel; steps with prompt portions run the mma.sync
            # prompt kernel
            tc = (ctx is not None and qkv.dtype == torch.bfloat16 and v_dim == head_dim and self.general_attention_tc
                  and self.lib.ullm_prefill_attention_supported(head_dim, num_q, num_kv)
                  and not (softcap > 0 and parts is not None))
            if (tc and ctx.decode_only and T == ctx.num_requests
                    and self.lib.ullm_decode_attention_supported(head_dim, num_q, num_kv)):
                self._decode_rows(qkv, out, k_pages, v_pages, block_table, req_slots, kv_len, num_q, num_kv, head_dim,
                                  page_size, window, scale, num_pages, False, ctx, None, keep_first, softcap, parts)
                return
            if (tc and keep_first == 0 and self.use_tcgen05_attention
                    and self.tc_attention_mode != "single" and qkv.stride(0) % head_dim == 0
                    and self.lib.ullm_prefill_attention_pair_supported(head_dim, num_q, num_kv, page_size)):
                # head size 128: the tcgen05 prompt kernel with two query tiles per block, with or without the cap,
                # or with every head's weights on every kv head's values
                args = (_ptr(qkv), qkv.stride(0), _ptr(parts if parts is not None else out), _ptr(k_pages), _ptr(v_pages),
                        _ptr(block_table), block_table.shape[1], _ptr(req_slots), _ptr(cu_q), _ptr(kv_len), T,
                        ctx.num_requests, num_q, num_kv, head_dim, page_size, int(window), float(scale), num_pages,
                        _ptr(self.status), _stream())
                if parts is not None:
                    code = self.lib.ullm_prefill_attention_pair_parts(*args)
                elif softcap > 0:
                    code = self.lib.ullm_prefill_attention_pair_capped(*args, float(softcap))
                else:
                    code = self.lib.ullm_prefill_attention_pair(*args)
                self._check(code, f"prefill_attention_pair (head_dim {head_dim}, cap {softcap})")
                self.prefill_attention_kernel = "pair"
                self.attention_path = "prefill_tcgen05"
                return
            if tc:
                self._check(self.lib.ullm_prefill_attention_ex(
                    _ptr(qkv), qkv.stride(0), _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                    block_table.shape[1], _ptr(req_slots), _ptr(cu_q), _ptr(kv_len), T, ctx.num_requests, num_q, num_kv,
                    head_dim, page_size, int(window), float(scale), num_pages, _ptr(self.status), _stream(),
                    int(keep_first), float(softcap), _ptr(parts)),
                    f"prefill_attention (head_dim {head_dim}, cap {softcap}, parts {parts is not None})")
                self.attention_path = "prefill"
                return
            self.attention_path = "generic"
            self._check(self.lib.ullm_paged_attention_generic_ex2(
                _DT[qkv.dtype], _ptr(qkv), qkv.stride(0), _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                block_table.shape[1], _ptr(req_slots), _ptr(cu_q), _ptr(kv_len), _ptr(token_req), T, num_q, num_kv,
                head_dim, page_size, int(window), float(scale), num_pages, _ptr(self.status), _stream(), v_dim,
                int(keep_first), float(softcap), _ptr(parts)),
                f"paged_attention (head_dim {head_dim}, values {v_dim}, cap {softcap}, parts {parts is not None})")
            return
        kept_tc = (keep_first > 0 and v_dim == head_dim and ctx is not None and qkv.dtype == torch.bfloat16
                   and fuse is None and self.lib.ullm_decode_attention_supported(head_dim, num_q, num_kv)
                   and self.lib.ullm_prefill_attention_supported(head_dim, num_q, num_kv))
        if kept_tc:
            # kept first positions on the tensor cores (head size 64 or 128): decode steps on the per-request split
            # kernel, steps with prompt portions on the mma.sync prompt kernel; both number a row's visible keys
            # "kept ones, then the window" and leave everything else as it is
            if ctx.decode_only and T == ctx.num_requests:
                self._decode_rows(qkv, out, k_pages, v_pages, block_table, req_slots, kv_len, num_q, num_kv, head_dim,
                                  page_size, window, scale, num_pages, False, ctx, None, keep_first)
                return
            self._check(self.lib.ullm_prefill_attention_kept(
                _ptr(qkv), qkv.stride(0), _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                block_table.shape[1], _ptr(req_slots), _ptr(cu_q), _ptr(kv_len), T, ctx.num_requests, num_q, num_kv,
                head_dim, page_size, int(window), float(scale), num_pages, _ptr(self.status), _stream(),
                int(keep_first)), f"prefill_attention (head_dim {head_dim}, first {keep_first} kept)")
            self.attention_path = "prefill"
            return
        if v_dim != head_dim or keep_first > 0:
            # values of a head size of their own, or kept first positions at other head sizes or in 32-bit: the
            # general kernel
            if fuse is not None:
                raise KernelError("paged_attention: q and k were left unprepared, but the general kernel takes this step")
            self.attention_path = "generic"
            self._check(self.lib.ullm_paged_attention_generic_ex(
                _DT[qkv.dtype], _ptr(qkv), qkv.stride(0), _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                block_table.shape[1], _ptr(req_slots), _ptr(cu_q), _ptr(kv_len), _ptr(token_req), T, num_q, num_kv,
                head_dim, page_size, int(window), float(scale), num_pages, _ptr(self.status), _stream(), v_dim,
                int(keep_first)), f"paged_attention (head_dim {head_dim}, values {v_dim}, first {keep_first} kept)")
            return
        decode_ok = (ctx is not None and qkv.dtype == torch.bfloat16
                     and self.lib.ullm_decode_attention_supported(head_dim, num_q, num_kv))
        if decode_ok and ctx.decode_only and T == ctx.num_requests:
            self._decode_rows(qkv, out, k_pages, v_pages, block_table, req_slots, kv_len, num_q, num_kv, head_dim,
                              page_size, window, scale, num_pages, ragged, ctx, fuse)
            return
        if fuse is not None:
            raise KernelError("paged_attention: q and k were left unprepared, but this step is no decode step")
        # A step that mixes decoded tokens with prompt portions: the one-token entries at its head (the scheduler
        # puts them first) go to the decode kernel, which streams their pages once; the prompt kernels would give
        # each of them a 128-row tile of its own.  The rest of the step follows with its own slices of the
        # per-request arrays (cu_q holds absolute rows, so q and out stay whole).
        n_dec = 0
        if decode_ok and self.mixed_decode_rows > 0 and getattr(ctx, "cu_q_host", None) is not None:
            cq = ctx.cu_q_host
            while n_dec < ctx.num_requests and cq[n_dec] == n_dec and cq[n_dec + 1] == n_dec + 1:
                n_dec += 1
            if n_dec < self.mixed_decode_rows or n_dec == ctx.num_requests:
                n_dec = 0
        if n_dec:
            lens = [ctx.start_positions_host[i] + 1 for i in range(n_dec)]
            ragged = n_dec > 1 and 2 * n_dec * max(lens) > 3 * sum(lens)
            self._decode_rows(qkv[:n_dec], out[:n_dec], k_pages, v_pages, block_table, req_slots[:n_dec], kv_len[:n_dec],
                              num_q, num_kv, head_dim, page_size, window, scale, num_pages, ragged, ctx)
            req_slots, cu_q, kv_len = req_slots[n_dec:], cu_q[n_dec:], kv_len[n_dec:]
        num_requests = (ctx.num_requests - n_dec) if ctx is not None else 0
        pair = single = False
        if ctx is not None and qkv.dtype == torch.bfloat16 and self.use_tcgen05_attention and qkv.stride(0) % head_dim == 0:
            pair = bool(self.tc_attention_mode != "single"
                        and self.lib.ullm_prefill_attention_pair_supported(head_dim, num_q, num_kv, page_size))
            single = bool(not pair and self.lib.ullm_prefill_attention_tcgen05_supported(head_dim, num_q, num_kv, page_size))
        if pair or single:
            entry = self.lib.ullm_prefill_attention_pair if pair else self.lib.ullm_prefill_attention_tcgen05
            self.prefill_attention_kernel = "pair" if pair else "single"
            self._check(entry(
                _ptr(qkv), qkv.stride(0), _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                block_table.shape[1], _ptr(req_slots), _ptr(cu_q), _ptr(kv_len), T, num_requests, num_q, num_kv,
                head_dim, page_size, int(window), float(scale), num_pages, _ptr(self.status), _stream()),
                f"prefill_attention_tcgen05 (head_dim {head_dim})")
            self.attention_path = "prefill_tcgen05"
            self.tcgen05_attention_blocks_per_sm = self.lib.ullm_prefill_attention_tcgen05_blocks_per_sm()
            return
        if (ctx is not None and qkv.dtype == torch.bfloat16
                and self.lib.ullm_prefill_attention_supported(head_dim, num_q, num_kv)):
            self._check(self.lib.ullm_prefill_attention(
                _ptr(qkv), qkv.stride(0), _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                block_table.shape[1], _ptr(req_slots), _ptr(cu_q), _ptr(kv_len), T, num_requests, num_q, num_kv,
                head_dim, page_size, int(window), float(scale), num_pages, _ptr(self.status), _stream()),
                f"prefill_attention (head_dim {head_dim})")
            self.attention_path = "prefill"
            return
        if n_dec:
            raise KernelError("paged_attention: a step's decode rows were split off but no prompt kernel takes the rest")
        self.attention_path = "generic"
        self._check(self.lib.ullm_paged_attention_generic(
            _DT[qkv.dtype], _ptr(qkv), qkv.stride(0), _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
            block_table.shape[1], _ptr(req_slots), _ptr(cu_q), _ptr(kv_len), _ptr(token_req), T, num_q, num_kv, head_dim, page_size,
            int(window), float(scale), num_pages, _ptr(self.status), _stream()),
            f"paged_attention (head_dim {head_dim})")

    @_timed("sampling")
    def argmax(self, logits, out):
        _need(logits, "logits", torch.float32, contiguous=False)
        _need(out, "out", torch.int32)
        R, V = logits.shape
        if logits.stride(1) != 1 or out.numel() < R:
            raise KernelError("argmax: logits rows must be contiguous and out must hold one id per row")
        self._check(self.lib.ullm_argmax(_ptr(logits), logits.stride(0), R, V, _ptr(out), _stream()), "argmax")

    def set_decode_cluster_merge(self, on: bool) -> None:
        """The splits of the per-request decode attention merge inside a cluster (True) or through scratch arrays
        and the merge kernel (False; tests compare the two), or "auto": the first for one or two requests."""
        self.decode_cluster_merge = on if on == "auto" else bool(on)

    def sample_force_one_block(self, on: bool) -> None:
        """Rows go to the one-block sampling kernel instead of the cluster kernel (tests compare the two)."""
        self.lib.ullm_sample_force_one_block(1 if on else 0)

    def sample_used_cluster(self) -> bool:
        return bool(self.lib.ullm_sample_last_used_cluster())

    @_timed("sampling")
    def sample(self, logits, temperature, top_k, top_p, min_p, uniform, out, probs_out=None, row_slots=None,
               last_tokens=None):
        _need(logits, "logits", torch.float32, contiguous=False)
        R, V = logits.shape
        if logits.stride(1) != 1:
            raise KernelError("sample: logits rows must be contiguous")
        for t, n, dt in ((temperature, "temperature", torch.float32), (top_k, "top_k", torch.int32),
                         (top_p, "top_p", torch.float32), (min_p, "min_p", torch.float32),
                         (uniform, "uniform", torch.float32), (out, "out", torch.int32)):
            _need(t, n, dt)
            if t.numel() < R:
                raise KernelError(f"sample: {n} holds {t.numel()} values for {R} rows")
        if probs_out is not None:
            _need(probs_out, "probs_out", torch.float32)
            if probs_out.shape != (R, V):
                raise KernelError("sample: probs_out must be [rows, vocab]")
        self._check(self.lib.ullm_sample(_ptr(logits), logits.stride(0), R, V, _ptr(temperature), _ptr(top_k),
                                         _ptr(top_p), _ptr(min_p), _ptr(uniform), _ptr(out), _ptr(probs_out),
                                         _ptr(row_slots), _ptr(last_tokens), _stream()), "sample")
