//! `include/dash_attn.h`, item for item: the structs `#[repr(C)]` field by field, every function of the
//! header in one `extern "C"` block.  All pointers but the parameter structs are device memory.
#![allow(non_camel_case_types)]

use core::ffi::{c_char, c_int, c_void};

/// `cudaStream_t`.
pub type dash_attn_stream_t = *mut c_void;

pub const DASH_ATTN_F32: i32 = 0;
pub const DASH_ATTN_BF16: i32 = 1;
pub const DASH_ATTN_F16: i32 = 2;

pub const DASH_ATTN_MASK_NONE: i32 = 0;
pub const DASH_ATTN_MASK_KEY_PADDING: i32 = 1;
pub const DASH_ATTN_MASK_PACKED: i32 = 2;

pub const DASH_ATTN_OK: c_int = 0;
pub const DASH_ATTN_INVALID: c_int = 1;
pub const DASH_ATTN_UNSUPPORTED: c_int = 2;
pub const DASH_ATTN_WORKSPACE: c_int = 3;
pub const DASH_ATTN_CUDA: c_int = 4;

/// A window side with no bound.
pub const DASH_ATTN_UNBOUNDED: i64 = -1;

pub const DASH_ATTN_PROBE_KERNEL_LAUNCHES: c_int = 0;
pub const DASH_ATTN_PROBE_BACKWARD_RUNS: c_int = 1;
pub const DASH_ATTN_PROBE_INPUT_COPIES: c_int = 2;
pub const DASH_ATTN_PROBE_ATOMIC_RUNS: c_int = 3;
pub const DASH_ATTN_PROBE_TENSOR_CORE_RUNS: c_int = 4;
pub const DASH_ATTN_PROBE_GENERIC_RUNS: c_int = 5;
pub const DASH_ATTN_PROBE_TENSOR_MAP_ENCODES: c_int = 6;

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct dash_attn_params {
    pub dtype: i32,
    pub b: i32,
    pub tq: i32,
    pub tk: i32,
    pub hq: i32,
    pub hkv: i32,
    pub d: i32,
    pub v_tk: i32,
    pub v_hkv: i32,
    pub v_d: i32,
    pub k_b: i32,
    pub k_d: i32,
    pub q_stride: [i64; 4],
    pub k_stride: [i64; 4],
    pub v_stride: [i64; 4],
    pub o_stride: [i64; 4],
    pub do_stride: [i64; 4],
    pub mask_kind: i32,
    pub key_padding: *const c_void,
    pub key_padding_elem_bytes: i32,
    pub key_padding_shape: [i32; 2],
    pub key_padding_stride: [i64; 2],
    pub cu_seqlens_q: *const c_void,
    pub cu_seqlens_k: *const c_void,
    pub cu_seqlens_q_len: i32,
    pub cu_seqlens_k_len: i32,
    pub index_elem_bytes: i32,
    pub causal: i32,
    pub has_window: i32,
    pub window_left: i64,
    pub window_right: i64,
    pub has_scale: i32,
    pub scale: f32,
    pub deterministic: i32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct dash_attn_decode_params {
    pub dtype: i32,
    pub b: i32,
    pub s: i32,
    pub hq: i32,
    pub hkv: i32,
    pub d: i32,
    pub k_b: i32,
    pub k_d: i32,
    pub v_b: i32,
    pub v_s: i32,
    pub v_hkv: i32,
    pub v_d: i32,
    pub q_stride: [i64; 3],
    pub k_stride: [i64; 4],
    pub v_stride: [i64; 4],
    pub lengths: *const c_void,
    pub lengths_len: i32,
    pub lengths_elem_bytes: i32,
    pub has_window: i32,
    pub window_left: i64,
    pub has_scale: i32,
    pub scale: f32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct dash_rope_tables {
    pub dtype: i32,
    pub dim: i32,
    pub len: i64,
    pub cos: *const c_void,
    pub sin: *const c_void,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct dash_rope_params {
    pub tokens: i64,
    pub d: i32,
    pub heads_a: i32,
    pub heads_b: i32,
    pub stride_a: [i64; 2],
    pub stride_b: [i64; 2],
    pub inverse: i32,
    pub positions: *const c_void,
    pub positions_elem_bytes: i32,
    pub cu_seqlens: *const c_void,
    pub cu_seqlens_len: i32,
    pub index_elem_bytes: i32,
    pub start: i64,
    pub period: i64,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct dash_sample_params {
    pub dtype: i32,
    pub b: i32,
    pub v: i32,
    pub row_stride: i64,
    pub temperature: f32,
    pub top_k: i64,
    pub top_p: f32,
    pub seed: u64,
    pub offset: u64,
    /// HOST memory.
    pub masked: *const u32,
    pub masked_len: i32,
    pub token_elem_bytes: i32,
}

extern "C" {
    pub fn dash_attn_forward_workspace(p: *const dash_attn_params) -> usize;
    pub fn dash_attn_backward_workspace(p: *const dash_attn_params) -> usize;
    pub fn dash_attn_decode_workspace(p: *const dash_attn_decode_params) -> usize;

    pub fn dash_attn_forward(
        p: *const dash_attn_params,
        q: *const c_void,
        k: *const c_void,
        v: *const c_void,
        o: *mut c_void,
        lse: *mut f32,
        workspace: *mut c_void,
        workspace_bytes: usize,
        stream: dash_attn_stream_t,
    ) -> c_int;

    pub fn dash_attn_backward(
        p: *const dash_attn_params,
        q: *const c_void,
        k: *const c_void,
        v: *const c_void,
        o: *const c_void,
        lse: *const f32,
        dout: *const c_void,
        dq: *mut c_void,
        dk: *mut c_void,
        dv: *mut c_void,
        workspace: *mut c_void,
        workspace_bytes: usize,
        stream: dash_attn_stream_t,
    ) -> c_int;

    pub fn dash_attn_decode(
        p: *const dash_attn_decode_params,
        q: *const c_void,
        k_cache: *const c_void,
        v_cache: *const c_void,
        out: *mut c_void,
        workspace: *mut c_void,
        workspace_bytes: usize,
        stream: dash_attn_stream_t,
    ) -> c_int;

    pub fn dash_attn_decode_append(
        p: *const dash_attn_decode_params,
        q: *const c_void,
        k_new: *const c_void,
        v_new: *const c_void,
        k_cache: *mut c_void,
        v_cache: *mut c_void,
        out: *mut c_void,
        workspace: *mut c_void,
        workspace_bytes: usize,
        stream: dash_attn_stream_t,
    ) -> c_int;

    pub fn dash_rope_apply(
        rope: *const dash_rope_tables,
        p: *const dash_rope_params,
        x_a: *const c_void,
        out_a: *mut c_void,
        x_b: *const c_void,
        out_b: *mut c_void,
        stream: dash_attn_stream_t,
    ) -> c_int;

    pub fn dash_attn_decode_append_rope_workspace(p: *const dash_attn_decode_params) -> usize;

    pub fn dash_attn_decode_append_rope(
        p: *const dash_attn_decode_params,
        rope: *const dash_rope_tables,
        positions: *const c_void,
        positions_elem_bytes: i32,
        q: *const c_void,
        k_new: *const c_void,
        v_new: *const c_void,
        k_cache: *mut c_void,
        v_cache: *mut c_void,
        out: *mut c_void,
        workspace: *mut c_void,
        workspace_bytes: usize,
        stream: dash_attn_stream_t,
    ) -> c_int;

    pub fn dash_sample_workspace(p: *const dash_sample_params) -> usize;

    pub fn dash_sample(
        p: *const dash_sample_params,
        logits: *const c_void,
        tokens: *mut c_void,
        logprob: *mut f32,
        tempered_logprob: *mut f32,
        sampling_logprob: *mut f32,
        workspace: *mut c_void,
        workspace_bytes: usize,
        stream: dash_attn_stream_t,
    ) -> c_int;

    pub fn dash_attn_decode_static(
        p: *const dash_attn_decode_params,
        q: *const c_void,
        k_cache: *const c_void,
        v_cache: *const c_void,
        out: *mut c_void,
        stream: dash_attn_stream_t,
    ) -> c_int;

    pub fn dash_attn_kernels_take(
        p: *const dash_attn_params,
        q: *const c_void,
        k: *const c_void,
        v: *const c_void,
        backward: c_int,
    ) -> c_int;

    pub fn dash_attn_device_status(clear: c_int) -> c_int;
    pub fn dash_attn_last_error() -> *const c_char;
    pub fn dash_attn_probe(which: c_int) -> u64;
    pub fn dash_attn_force_generic(on: c_int);
    pub fn dash_attn_force_tensor(on: c_int);
}
