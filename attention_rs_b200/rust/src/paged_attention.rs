//! The dispatch part of `PagedAttention::cuda_fwd_t` rewritten for libpagedattention_b200
//! (replaces src/paged_attention.rs:154-236 of the reference; the shape checks above it stay as they
//! are).  NOT COMPILED in the environment this repository was developed in.
//!
//! Differences from the reference's dispatch:
//!  * the v1 / v2 choice is asked of the library (`pa_paged_attention_uses_partitions`) instead of the
//!    `num_seqs * num_heads > 512` rule, which was tuned for one CTA per query head;
//!  * `self.alibi_slopes` is finally passed down (the reference's CUDA path drops it);
//!  * a `u8` cache selects the FP8-E4M3 mode with `k_scale` / `v_scale`;
//!  * the status code is turned into a `candle::Error`.
//!
//! ```ignore
//! let use_v2 = unsafe {
//!     kernels::ffi::pa_paged_attention_uses_partitions(
//!         num_seqs as i64, num_heads as i64, num_kv_heads as i64, self.max_context_len as i64) != 0
//! };
//! let alibi_ptr = match &self.alibi_slopes {
//!     Some(t) => { /* storage_and_layout(), as_cuda_slice::<f32>() as for the other tensors */ ptr }
//!     None => std::ptr::null(),
//! };
//! let kv_dtype = if self.key_cache.dtype() == DType::U8 { 3 } else { internal_type };
//! let rc = if !use_v2 {
//!     unsafe { kernels::ffi::paged_attention_v1_ex(out_ptr, q_ptr, kc_ptr, vc_ptr, num_kv_heads as c_int,
//!         self.softmax_scale, bt_ptr, cl_ptr, block_size as c_int, self.max_context_len as c_int,
//!         num_seqs as c_int, num_heads as c_int, head_size as c_int, max_num_blocks_per_seq as c_int,
//!         q_stride as c_int, kv_block_stride as c_int, kv_head_stride as c_int, internal_type,
//!         self.softcapping, alibi_ptr, kv_dtype, self.k_scale, self.v_scale, *dev.cu_stream() as i64) }
//! } else {
//!     // tmp_out / exp_sums / max_logits allocated exactly as at src/paged_attention.rs:199-203
//!     unsafe { kernels::ffi::paged_attention_v2_ex(out_ptr, exp_sums_ptr, max_logits_ptr, tmp_out_ptr, /* same tail */) }
//! };
//! if rc != 0 {
//!     let msg = unsafe { std::ffi::CStr::from_ptr(kernels::ffi::pa_last_error()) }.to_string_lossy();
//!     candle::bail!("paged-attention: {msg}")
//! }
//! ```
