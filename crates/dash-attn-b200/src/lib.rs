//! dash-ops' attention on NVIDIA B200 (compute capability 10.0): the [`AttentionBackend`] of Burn's CUDA
//! backend, every method a call through the C ABI of `include/dash_attn.h` on Burn-owned buffers.
//!
//! NOT COMPILED where this was written (no Rust toolchain there).  It replaces
//! `crates/dash-ops/src/attention/cube.rs:1232-1337` for devices this library takes; everything above
//! the backend extension - dash-ops' public functions (`attention.rs:648-806`), the `Autodiff` node
//! (`:377-456`), the routing of a tracked decoding step (`:498-542`), dash-mag's gateway - stays as it
//! is and reaches these methods through Burn's dispatch.
//!
//! There is no CubeCL kernel, no other backend and no CPU fallback on this path: a call the library
//! refuses panics with the library's message where dash-ops panics (shapes that do not fit together)
//! and with "unsupported" otherwise.
pub mod ffi;

use std::ffi::{c_void, CStr};

use burn::backend::tensor::{BoolTensor, FloatTensor, IntTensor};
use burn::backend::{DType, Shape};
use burn_cubecl::ops::numeric::empty_device_contiguous_dtype;
use burn_cubecl::tensor::CubeTensor;
use burn_cubecl::CubeBackend;
use dash_contract::attention::AttentionOptions;
use dash_ops::attention::{AttentionBackend, AttentionMaskPrimitive, CacheLengths};

use ffi::*;

/// The raw device address of a tensor's first element: the handle's resource as CubeCL's CUDA server
/// hands it out (`patches/cubecl-cuda/src/compute/server.rs:1357-1368`, `GpuResource { ptr, size }`),
/// plus the handle's offset.  Taking it also orders the call behind every pending write of the buffer.
fn device_ptr(tensor: &CubeTensor) -> *mut c_void {
    let binding = tensor.handle.clone().binding();
    let resource = tensor.client.get_resource(binding).expect("attention: a buffer whose producer failed");
    resource.resource().ptr as *mut c_void
}

/// The CUDA stream the calling thread's CubeCL work is enqueued on (`compute/stream.rs`): the library
/// enqueues behind it and returns without synchronising.
fn stream_of(tensor: &CubeTensor) -> dash_attn_stream_t {
    tensor.client.cuda_stream() as dash_attn_stream_t
}

fn dtype_code(dtype: DType) -> i32 {
    match dtype {
        DType::F32 => DASH_ATTN_F32,
        DType::BF16 => DASH_ATTN_BF16,
        DType::F16 => DASH_ATTN_F16,
        other => panic!("attention: the dtype must be f32, bf16 or f16, got {other:?}"),
    }
}

fn dims<const N: usize>(tensor: &CubeTensor, what: &str) -> [i32; N] {
    let shape = tensor.meta.shape();
    assert_eq!(shape.num_dims(), N, "{what}");
    core::array::from_fn(|i| i32::try_from(shape[i]).expect("attention: a dimension beyond i32"))
}

/// Strides in ELEMENTS, as the header wants them; a tiled (matmul-storage) tensor is untiled first by
/// the caller, as `cube.rs:444-452` does.
fn strides<const N: usize>(tensor: &CubeTensor) -> [i64; N] {
    let strides = tensor.meta.strides();
    core::array::from_fn(|i| strides[i] as i64)
}

fn int_bytes(dtype: DType, what: &str) -> i32 {
    match dtype {
        DType::I32 | DType::U32 => 4,
        DType::I64 | DType::U64 => 8,
        other => panic!("{what} hold 4- or 8-byte integers, got {other:?}"),
    }
}

/// Turns a status into dash-ops' behaviour: a panic with the library's own words.
fn check(op: &str, code: i32) {
    if code == DASH_ATTN_OK {
        return;
    }
    // SAFETY: a NUL-terminated string owned by the library, valid until this thread's next call.
    let message = unsafe { CStr::from_ptr(dash_attn_last_error()) }.to_string_lossy().into_owned();
    match code {
        DASH_ATTN_INVALID => panic!("{message}"),
        DASH_ATTN_UNSUPPORTED => panic!("unsupported: {message}"),
        _ => panic!("{op}: {message}"),
    }
}

fn scratch(like: &CubeTensor, bytes: usize) -> Option<CubeTensor> {
    (bytes > 0).then(|| {
        empty_device_contiguous_dtype(like.client.clone(), like.device.clone(), Shape::new([bytes.div_ceil(4)]), DType::F32)
    })
}

/// `dash_attn_params` of a training call.  The mask's tensors are read in place: offsets `i32` or
/// `i64`, the padding mask one byte or four per key (so the casts of `cube.rs:476-483,535-542` go).
fn train_params(
    query: &CubeTensor,
    key: &CubeTensor,
    value: &CubeTensor,
    mask: &AttentionMaskPrimitive<CubeBackend>,
    options: &AttentionOptions,
) -> dash_attn_params {
    let [b, tq, hq, d] = dims::<4>(query, "attention: query is [B, Tq, Hq, D]");
    let [k_b, tk, hkv, k_d] = dims::<4>(key, "attention: key is [B, Tk, Hkv, D]");
    let [_, v_tk, v_hkv, v_d] = dims::<4>(value, "attention: key and value must have one shape");
    assert!(key.dtype == query.dtype && value.dtype == query.dtype, "attention: queries, keys and values share one dtype");
    let mut p = dash_attn_params {
        dtype: dtype_code(query.dtype),
        b,
        tq,
        tk,
        hq,
        hkv,
        d,
        v_tk,
        v_hkv,
        v_d,
        k_b,
        k_d,
        q_stride: strides::<4>(query),
        k_stride: strides::<4>(key),
        v_stride: strides::<4>(value),
        o_stride: [0; 4],
        do_stride: [0; 4],
        mask_kind: DASH_ATTN_MASK_NONE,
        key_padding: core::ptr::null(),
        key_padding_elem_bytes: 0,
        key_padding_shape: [0; 2],
        key_padding_stride: [0; 2],
        cu_seqlens_q: core::ptr::null(),
        cu_seqlens_k: core::ptr::null(),
        cu_seqlens_q_len: 0,
        cu_seqlens_k_len: 0,
        index_elem_bytes: 0,
        causal: options.causal as i32,
        has_window: options.window.is_some() as i32,
        window_left: DASH_ATTN_UNBOUNDED,
        window_right: DASH_ATTN_UNBOUNDED,
        has_scale: options.scale.is_some() as i32,
        scale: options.scale.unwrap_or(0.0),
        deterministic: options.deterministic as i32,
    };
    if let Some(window) = options.window {
        let side = |x: usize| if x == usize::MAX { DASH_ATTN_UNBOUNDED } else { x as i64 };
        p.window_left = side(window.left);
        p.window_right = side(window.right);
    }
    match mask {
        AttentionMaskPrimitive::None => {}
        AttentionMaskPrimitive::KeyPadding(padding) => {
            p.mask_kind = DASH_ATTN_MASK_KEY_PADDING;
            p.key_padding = device_ptr(padding);
            p.key_padding_elem_bytes = padding.dtype.size() as i32;
            p.key_padding_shape = dims::<2>(padding, "attention: the key padding mask is [B, Tk]");
            p.key_padding_stride = strides::<2>(padding);
        }
        AttentionMaskPrimitive::Packed { cu_seqlens_q, cu_seqlens_k } => {
            assert_eq!(cu_seqlens_q.dtype, cu_seqlens_k.dtype, "attention: cu_seqlens_q and cu_seqlens_k share one integer type");
            p.mask_kind = DASH_ATTN_MASK_PACKED;
            p.cu_seqlens_q = device_ptr(cu_seqlens_q);
            p.cu_seqlens_k = device_ptr(cu_seqlens_k);
            p.cu_seqlens_q_len = dims::<1>(cu_seqlens_q, "attention: cu_seqlens_q is [S + 1]")[0];
            p.cu_seqlens_k_len = dims::<1>(cu_seqlens_k, "attention: cu_seqlens_k is [S + 1]")[0];
            p.index_elem_bytes = int_bytes(cu_seqlens_q.dtype, "attention: cu_seqlens");
        }
    }
    p
}

impl AttentionBackend for CubeBackend {
    fn attention_forward(
        query: FloatTensor<Self>,
        key: FloatTensor<Self>,
        value: FloatTensor<Self>,
        mask: AttentionMaskPrimitive<Self>,
        options: AttentionOptions,
    ) -> (FloatTensor<Self>, FloatTensor<Self>) {
        let p = train_params(&query, &key, &value, &mask, &options);
        let (client, device) = (query.client.clone(), query.device.clone());
        // Outputs as the reference's launch glue allocates them (cube.rs:573-580): contiguous.
        let shape = [p.b as usize, p.tq as usize, p.hq as usize, p.d as usize];
        let output = empty_device_contiguous_dtype(client.clone(), device.clone(), Shape::new(shape), query.dtype);
        let lse = empty_device_contiguous_dtype(client, device, Shape::new([shape[0], shape[1], shape[2]]), DType::F32);
        // SAFETY: the parameters describe the tensors whose addresses are passed; the outputs and the
        // workspace are fresh allocations of the sizes the library asks for; everything stays alive
        // until the stream has run the call because Burn frees a buffer behind the stream's work.
        let code = unsafe {
            let ws = scratch(&query, dash_attn_forward_workspace(&p));
            dash_attn_forward(
                &p,
                device_ptr(&query),
                device_ptr(&key),
                device_ptr(&value),
                device_ptr(&output),
                device_ptr(&lse) as *mut f32,
                ws.as_ref().map_or(core::ptr::null_mut(), device_ptr),
                ws.as_ref().map_or(0, |w| w.meta.shape()[0] * 4),
                stream_of(&query),
            )
        };
        check("attention", code);
        (output, lse)
    }

    fn attention_backward(
        query: FloatTensor<Self>,
        key: FloatTensor<Self>,
        value: FloatTensor<Self>,
        output: FloatTensor<Self>,
        lse: FloatTensor<Self>,
        grad_output: FloatTensor<Self>,
        mask: AttentionMaskPrimitive<Self>,
        options: AttentionOptions,
    ) -> (FloatTensor<Self>, FloatTensor<Self>, FloatTensor<Self>) {
        let mut p = train_params(&query, &key, &value, &mask, &options);
        // attention.rs:689-724: the same three checks, the same words.
        assert_eq!(output.meta.shape(), query.meta.shape(), "attention_backward: output");
        assert_eq!(grad_output.meta.shape(), query.meta.shape(), "attention_backward: grad");
        assert_eq!(dims::<3>(&lse, "attention_backward: lse"), [p.b, p.tq, p.hq], "attention_backward: lse");
        p.o_stride = strides::<4>(&output);
        p.do_stride = strides::<4>(&grad_output);
        // The log-sum-exp is read contiguous (it is the forward's own output).
        let lse = burn_cubecl::kernel::into_contiguous(lse);
        let (client, device) = (query.client.clone(), query.device.clone());
        let like = |t: &CubeTensor| empty_device_contiguous_dtype(client.clone(), device.clone(), t.meta.shape().clone(), t.dtype);
        let (grad_query, grad_key, grad_value) = (like(&query), like(&key), like(&value));
        // SAFETY: as in the forward.
        let code = unsafe {
            let ws = scratch(&query, dash_attn_backward_workspace(&p));
            dash_attn_backward(
                &p,
                device_ptr(&query),
                device_ptr(&key),
                device_ptr(&value),
                device_ptr(&output),
                device_ptr(&lse) as *const f32,
                device_ptr(&grad_output),
                device_ptr(&grad_query),
                device_ptr(&grad_key),
                device_ptr(&grad_value),
                ws.as_ref().map_or(core::ptr::null_mut(), device_ptr),
                ws.as_ref().map_or(0, |w| w.meta.shape()[0] * 4),
                stream_of(&query),
            )
        };
        check("attention_backward", code);
        (grad_query, grad_key, grad_value)
    }

    fn attention_decode(
        query: FloatTensor<Self>,
        key: FloatTensor<Self>,
        value: FloatTensor<Self>,
        lengths: CacheLengths<Self>,
        options: AttentionOptions,
    ) -> FloatTensor<Self> {
        let [b, hq, d] = dims::<3>(&query, "attention_decode: query is [B, Hq, D]");
        let [k_b, s, hkv, k_d] = dims::<4>(&key, "attention_decode: key is [B, S, Hkv, D]");
        let [v_b, v_s, v_hkv, v_d] = dims::<4>(&value, "attention: key and value must have one shape");
        assert!(key.dtype == query.dtype && value.dtype == query.dtype, "attention_decode: queries, keys and values share one dtype");
        let mut p = dash_attn_decode_params {
            dtype: dtype_code(query.dtype),
            b,
            s,
            hq,
            hkv,
            d,
            k_b,
            k_d,
            v_b,
            v_s,
            v_hkv,
            v_d,
            q_stride: strides::<3>(&query),
            k_stride: strides::<4>(&key),   // a slice of a longer cache is read in place
            v_stride: strides::<4>(&value),
            lengths: core::ptr::null(),
            lengths_len: 0,
            lengths_elem_bytes: 0,
            has_window: options.window.is_some() as i32,
            window_left: DASH_ATTN_UNBOUNDED,
            has_scale: options.scale.is_some() as i32,
            scale: options.scale.unwrap_or(0.0),
        };
        if let Some(window) = options.window {
            p.window_left = if window.left == usize::MAX { DASH_ATTN_UNBOUNDED } else { window.left as i64 };
        }
        let lengths = match lengths {
            CacheLengths::Full => None,
            CacheLengths::Lengths(lengths) => Some(burn_cubecl::kernel::into_contiguous(lengths)),
        };
        if let Some(lengths) = &lengths {
            p.lengths = device_ptr(lengths);
            p.lengths_len = dims::<1>(lengths, "attention_decode: the cache lengths are [B]")[0];
            p.lengths_elem_bytes = int_bytes(lengths.dtype, "attention_decode: the cache lengths");
        }
        let output = empty_device_contiguous_dtype(
            query.client.clone(),
            query.device.clone(),
            Shape::new([b as usize, hq as usize, d as usize]),
            query.dtype,
        );
        // SAFETY: as in the forward.
        let code = unsafe {
            let ws = scratch(&query, dash_attn_decode_workspace(&p));
            dash_attn_decode(
                &p,
                device_ptr(&query),
                device_ptr(&key),
                device_ptr(&value),
                device_ptr(&output),
                ws.as_ref().map_or(core::ptr::null_mut(), device_ptr),
                ws.as_ref().map_or(0, |w| w.meta.shape()[0] * 4),
                stream_of(&query),
            )
        };
        check("attention_decode", code);
        output
    }
}

/// dash-ops' `probe` counters (`attention.rs:158-221`) read from the library.
pub mod probe {
    use super::ffi::*;

    pub fn kernel_launches() -> u64 {
        unsafe { dash_attn_probe(DASH_ATTN_PROBE_KERNEL_LAUNCHES) }
    }
    pub fn backward_runs() -> u64 {
        unsafe { dash_attn_probe(DASH_ATTN_PROBE_BACKWARD_RUNS) }
    }
    /// Always 0: every input is read in place.
    pub fn input_copies() -> u64 {
        unsafe { dash_attn_probe(DASH_ATTN_PROBE_INPUT_COPIES) }
    }
    pub fn atomic_runs() -> u64 {
        unsafe { dash_attn_probe(DASH_ATTN_PROBE_ATOMIC_RUNS) }
    }
}

/// Whether the tensor-core kernels take a call (`kernels_take`, `attention.rs:814-821`).
pub fn kernels_take(
    query: &CubeTensor,
    key: &CubeTensor,
    value: &CubeTensor,
    mask: &AttentionMaskPrimitive<CubeBackend>,
    options: &AttentionOptions,
    backward: bool,
) -> bool {
    let p = train_params(query, key, value, mask, options);
    unsafe { dash_attn_kernels_take(&p, device_ptr(query), device_ptr(key), device_ptr(value), backward as i32) == 1 }
}

// The steps either side of the decoding step (dash_rope_apply, dash_attn_decode_append[_rope],
// dash_sample, dash_attn_decode_static) are declared in `ffi` and bound the same way from dash-mag's
// `Rope` (crates/dash-mag/src/rope.rs), its cache update (crates/dash-mag/src/tensor.rs:732-744) and
// dash-ops' `sample` (crates/dash-ops/src/sample.rs): parameters from the tensors' shapes and strides,
// outputs allocated contiguous, the workspace from the matching `*_workspace` query.
#[allow(unused)]
fn _types_used(_: BoolTensor<CubeBackend>, _: IntTensor<CubeBackend>) {}
