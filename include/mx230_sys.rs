// Generated from mx230_attn.h by gen_rust_extern.py; link with `-l dylib=mx230_attn`.
#![allow(non_camel_case_types, dead_code)]
use std::ffi::{c_char, c_int, c_longlong, c_uint, c_void};
#[repr(C)] pub struct Mx230Handle { _p: [u8; 0] }
#[repr(C)] pub struct Mx230KvPool { _p: [u8; 0] }
#[repr(C)] pub struct Mx230Sched { _p: [u8; 0] }
#[repr(C)] pub struct Mx230SplitKvComm { _p: [u8; 0] }
extern "C" {
    pub fn mx230_abi_version() -> c_int;
    pub fn mx230_last_error() -> *const c_char;
    pub fn mx230_status_string(code: c_int) -> *const c_char;
    pub fn mx230_create(out: *mut *mut Mx230Handle, device: c_int, workspace_bytes: usize) -> c_int;
    pub fn mx230_destroy(h: *mut Mx230Handle) -> c_int;
    pub fn mx230_reserve(h: *mut Mx230Handle, bytes: usize) -> c_int;
    pub fn mx230_set_option(h: *mut Mx230Handle, option: c_int, value: c_int) -> c_int;
    pub fn mx230_flash_workspace_bytes(batch_heads: c_int, n: c_int, with_backward: c_int) -> usize;
    pub fn mx230_decode_workspace_bytes(n_seq: c_int, n_head: c_int, max_splits: c_int) -> usize;
    pub fn mx230_check_status(h: *mut Mx230Handle, stream: *mut c_void) -> c_int;
    pub fn mx230_launch_count(h: *const Mx230Handle) -> c_longlong;
    pub fn mx230_pseudo_rand(out_host: *mut f32, n: usize, seed: u64) -> c_int;
    pub fn mx230_fill_normal(out_host: *mut f32, n: usize, seed: u64, tensor_index: u64) -> c_int;
    pub fn mx230_profile_enable(h: *mut Mx230Handle, on: c_int) -> c_int;
    pub fn mx230_profile_reset(h: *mut Mx230Handle) -> c_int;
    pub fn mx230_profile_read(
        h: *mut Mx230Handle, kernel: c_int, launches: *mut c_longlong, total_ms: *mut f64,
    ) -> c_int;
    pub fn mx230_kernel_name(kernel: c_int) -> *const c_char;
    pub fn mx230_attn_flash(
        h: *mut Mx230Handle, stream: *mut c_void, Q: *const f32, K: *const f32, V: *const f32, O: *mut f32,
        batch_heads: c_int, n: c_int, causal: c_int,
    ) -> c_int;
    pub fn mx230_attn_flash_lse(
        h: *mut Mx230Handle, stream: *mut c_void, Q: *const f32, K: *const f32, V: *const f32, O: *mut f32,
        L: *mut f32, batch_heads: c_int, n: c_int, causal: c_int,
    ) -> c_int;
    pub fn mx230_attn_bwd_preprocess(
        h: *mut Mx230Handle, stream: *mut c_void, dO: *const f32, O: *const f32, Delta: *mut f32,
        batch_heads: c_int, n: c_int,
    ) -> c_int;
    pub fn mx230_attn_bwd_dq(
        h: *mut Mx230Handle, stream: *mut c_void, Q: *const f32, K: *const f32, V: *const f32, dO: *const f32,
        L: *const f32, Delta: *const f32, dQ: *mut f32, batch_heads: c_int, n: c_int, causal: c_int,
    ) -> c_int;
    pub fn mx230_attn_bwd_dkv(
        h: *mut Mx230Handle, stream: *mut c_void, Q: *const f32, K: *const f32, V: *const f32, dO: *const f32,
        L: *const f32, Delta: *const f32, dK: *mut f32, dV: *mut f32, batch_heads: c_int, n: c_int, causal: c_int,
    ) -> c_int;
    pub fn mx230_attn_bwd_flash(
        h: *mut Mx230Handle, stream: *mut c_void, Q: *const f32, K: *const f32, V: *const f32, dO: *const f32,
        L: *const f32, Delta: *const f32, dQ: *mut f32, dK: *mut f32, dV: *mut f32, batch_heads: c_int, n: c_int,
        causal: c_int,
    ) -> c_int;
    pub fn mx230_cast_bf16(
        h: *mut Mx230Handle, stream: *mut c_void, src: *const f32, dst_bf16: *mut c_void, count: usize,
    ) -> c_int;
    pub fn mx230_attn_flash_bf16(
        h: *mut Mx230Handle, stream: *mut c_void, Qb: *const c_void, Kb: *const c_void, Vb: *const c_void,
        O: *mut f32, L_or_null: *mut f32, batch_heads: c_int, n: c_int, causal: c_int,
    ) -> c_int;
    pub fn mx230_attn_bwd_flash_bf16(
        h: *mut Mx230Handle, stream: *mut c_void, Qb: *const c_void, Kb: *const c_void, Vb: *const c_void,
        dOb: *const c_void, L: *const f32, Delta: *const f32, dQ: *mut f32, dK: *mut f32, dV: *mut f32,
        batch_heads: c_int, n: c_int, causal: c_int,
    ) -> c_int;
    pub fn mx230_rope(
        h: *mut Mx230Handle, stream: *mut c_void, qkv: *mut f32, pos: c_int, n_head: c_int, n_kv_head: c_int,
        head_dim: c_int, theta: f32,
    ) -> c_int;
    pub fn mx230_rope_dyn(
        h: *mut Mx230Handle, stream: *mut c_void, qkv: *mut f32, pos_ptr: *const c_int, n_head: c_int,
        n_kv_head: c_int, head_dim: c_int, theta: f32,
    ) -> c_int;
    pub fn mx230_rope_batch(
        h: *mut Mx230Handle, stream: *mut c_void, qkv: *mut f32, pos0: c_int, n_tok: c_int, n_head: c_int,
        n_kv_head: c_int, head_dim: c_int, stride: c_int, theta: f32,
    ) -> c_int;
    pub fn mx230_rope_seqpos(
        h: *mut Mx230Handle, stream: *mut c_void, qkv: *mut f32, pos: *const c_int, n_seq: c_int, n_head: c_int,
        n_kv_head: c_int, head_dim: c_int, stride: c_int, theta: f32,
    ) -> c_int;
    pub fn mx230_copy_kv(
        h: *mut Mx230Handle, stream: *mut c_void, kcache: *mut f32, vcache: *mut f32, qkv: *const f32, pos: c_int,
        q_dim: c_int, kv_dim: c_int,
    ) -> c_int;
    pub fn mx230_copy_kv_dyn(
        h: *mut Mx230Handle, stream: *mut c_void, kcache: *mut f32, vcache: *mut f32, qkv: *const f32,
        pos_ptr: *const c_int, q_dim: c_int, kv_dim: c_int,
    ) -> c_int;
    pub fn mx230_copy_kv_paged_dyn(
        h: *mut Mx230Handle, stream: *mut c_void, kcache: *mut f32, vcache: *mut f32, qkv: *const f32,
        pos_ptr: *const c_int, q_dim: c_int, kv_dim: c_int, bt: *const c_int, bs: c_int,
    ) -> c_int;
    pub fn mx230_copy_kv_batch(
        h: *mut Mx230Handle, stream: *mut c_void, kcache: *mut f32, vcache: *mut f32, qkv: *const f32, pos0: c_int,
        n_tok: c_int, q_dim: c_int, kv_dim: c_int, stride: c_int,
    ) -> c_int;
    pub fn mx230_copy_kv_batch_paged(
        h: *mut Mx230Handle, stream: *mut c_void, kcache: *mut f32, vcache: *mut f32, qkv: *const f32, pos0: c_int,
        n_tok: c_int, q_dim: c_int, kv_dim: c_int, stride: c_int, bt: *const c_int, bs: c_int,
    ) -> c_int;
    pub fn mx230_copy_kv_seqpos(
        h: *mut Mx230Handle, stream: *mut c_void, kcache: *mut f32, vcache: *mut f32, qkv: *const f32,
        pos: *const c_int, n_seq: c_int, q_dim: c_int, kv_dim: c_int, qkv_stride: c_int, tables: *const c_int,
        block_size: c_int, n_log: c_int,
    ) -> c_int;
    pub fn mx230_quantize_kv(
        h: *mut Mx230Handle, stream: *mut c_void, kq: *mut i8, vq: *mut i8, ks: *mut f32, vs: *mut f32,
        kb: *mut f32, vb: *mut f32, qkv: *const f32, pos: c_int, q_dim: c_int, n_kv_head: c_int, head_dim: c_int,
    ) -> c_int;
    pub fn mx230_quantize_kv_dyn(
        h: *mut Mx230Handle, stream: *mut c_void, kq: *mut i8, vq: *mut i8, ks: *mut f32, vs: *mut f32,
        kb: *mut f32, vb: *mut f32, qkv: *const f32, pos_ptr: *const c_int, q_dim: c_int, n_kv_head: c_int,
        head_dim: c_int,
    ) -> c_int;
    pub fn mx230_quantize_kv_paged_dyn(
        h: *mut Mx230Handle, stream: *mut c_void, kq: *mut i8, vq: *mut i8, ks: *mut f32, vs: *mut f32,
        kb: *mut f32, vb: *mut f32, qkv: *const f32, pos_ptr: *const c_int, q_dim: c_int, n_kv_head: c_int,
        head_dim: c_int, bt: *const c_int, bs: c_int,
    ) -> c_int;
    pub fn mx230_quantize_kv_batch(
        h: *mut Mx230Handle, stream: *mut c_void, kq: *mut i8, vq: *mut i8, ks: *mut f32, vs: *mut f32,
        kb: *mut f32, vb: *mut f32, qkv: *const f32, pos0: c_int, n_tok: c_int, q_dim: c_int, n_kv_head: c_int,
        head_dim: c_int, stride: c_int,
    ) -> c_int;
    pub fn mx230_quantize_kv_batch_paged(
        h: *mut Mx230Handle, stream: *mut c_void, kq: *mut i8, vq: *mut i8, ks: *mut f32, vs: *mut f32,
        kb: *mut f32, vb: *mut f32, qkv: *const f32, pos0: c_int, n_tok: c_int, q_dim: c_int, n_kv_head: c_int,
        head_dim: c_int, stride: c_int, bt: *const c_int, bs: c_int,
    ) -> c_int;
    pub fn mx230_quantize_kv_seqpos(
        h: *mut Mx230Handle, stream: *mut c_void, kq: *mut i8, vq: *mut i8, ks: *mut f32, vs: *mut f32,
        kb: *mut f32, vb: *mut f32, qkv: *const f32, pos: *const c_int, n_seq: c_int, q_dim: c_int,
        n_kv_head: c_int, head_dim: c_int, qkv_stride: c_int, tables: *const c_int, block_size: c_int, n_log: c_int,
    ) -> c_int;
    pub fn mx230_attn_decode(
        h: *mut Mx230Handle, stream: *mut c_void, out: *mut f32, qkv: *const f32, kcache: *const f32,
        vcache: *const f32, t_cur: c_int, n_head: c_int, n_kv_head: c_int, head_dim: c_int,
    ) -> c_int;
    pub fn mx230_attn_decode_dyn(
        h: *mut Mx230Handle, stream: *mut c_void, out: *mut f32, qkv: *const f32, kcache: *const f32,
        vcache: *const f32, pos_ptr: *const c_int, n_head: c_int, n_kv_head: c_int, head_dim: c_int,
    ) -> c_int;
    pub fn mx230_attn_decode_paged(
        h: *mut Mx230Handle, stream: *mut c_void, out: *mut f32, qkv: *const f32, kcache: *const f32,
        vcache: *const f32, t_cur: c_int, n_head: c_int, n_kv_head: c_int, head_dim: c_int, bt: *const c_int,
        bs: c_int,
    ) -> c_int;
    pub fn mx230_attn_decode_paged_dyn(
        h: *mut Mx230Handle, stream: *mut c_void, out: *mut f32, qkv: *const f32, kcache: *const f32,
        vcache: *const f32, pos_ptr: *const c_int, n_head: c_int, n_kv_head: c_int, head_dim: c_int,
        bt: *const c_int, bs: c_int,
    ) -> c_int;
    pub fn mx230_attn_decode_batched(
        h: *mut Mx230Handle, stream: *mut c_void, out: *mut f32, qkv: *const f32, kcache: *const f32,
        vcache: *const f32, pos: *const c_int, n_seq: c_int, n_head: c_int, n_kv_head: c_int, head_dim: c_int,
        tables: *const c_int, block_size: c_int, n_log: c_int, qkv_stride: c_int, out_stride: c_int,
    ) -> c_int;
    pub fn mx230_attn_decode_q8(
        h: *mut Mx230Handle, stream: *mut c_void, out: *mut f32, qkv: *const f32, kq: *const i8, vq: *const i8,
        ks: *const f32, vs: *const f32, kb: *const f32, vb: *const f32, t_cur: c_int, n_head: c_int,
        n_kv_head: c_int, head_dim: c_int,
    ) -> c_int;
    pub fn mx230_attn_decode_q8_dyn(
        h: *mut Mx230Handle, stream: *mut c_void, out: *mut f32, qkv: *const f32, kq: *const i8, vq: *const i8,
        ks: *const f32, vs: *const f32, kb: *const f32, vb: *const f32, pos_ptr: *const c_int, n_head: c_int,
        n_kv_head: c_int, head_dim: c_int,
    ) -> c_int;
    pub fn mx230_attn_decode_q8_paged(
        h: *mut Mx230Handle, stream: *mut c_void, out: *mut f32, qkv: *const f32, kq: *const i8, vq: *const i8,
        ks: *const f32, vs: *const f32, kb: *const f32, vb: *const f32, t_cur: c_int, n_head: c_int,
        n_kv_head: c_int, head_dim: c_int, bt: *const c_int, bs: c_int,
    ) -> c_int;
    pub fn mx230_attn_decode_q8_paged_dyn(
        h: *mut Mx230Handle, stream: *mut c_void, out: *mut f32, qkv: *const f32, kq: *const i8, vq: *const i8,
        ks: *const f32, vs: *const f32, kb: *const f32, vb: *const f32, pos_ptr: *const c_int, n_head: c_int,
        n_kv_head: c_int, head_dim: c_int, bt: *const c_int, bs: c_int,
    ) -> c_int;
    pub fn mx230_attn_decode_q8_batched(
        h: *mut Mx230Handle, stream: *mut c_void, out: *mut f32, qkv: *const f32, kq: *const i8, vq: *const i8,
        ks: *const f32, vs: *const f32, kb: *const f32, vb: *const f32, pos: *const c_int, n_seq: c_int,
        n_head: c_int, n_kv_head: c_int, head_dim: c_int, tables: *const c_int, block_size: c_int, n_log: c_int,
        qkv_stride: c_int, out_stride: c_int,
    ) -> c_int;
    pub fn mx230_attn_decode_q8_noalloc(
        stream: *mut c_void, out: *mut f32, qkv: *const f32, kq: *const i8, vq: *const i8, ks: *const f32,
        vs: *const f32, kb: *const f32, vb: *const f32, t_cur: c_int, n_head: c_int, n_kv_head: c_int,
        head_dim: c_int,
    ) -> c_int;
    pub fn mx230_attn_decode_slab(
        h: *mut Mx230Handle, stream: *mut c_void, out: *mut f32, qkv: *const f32, kcache: *const f32,
        vcache: *const f32, kq: *const i8, vq: *const i8, ks: *const f32, vs: *const f32, kb: *const f32,
        vb: *const f32, pos: *const c_int, n_seq: c_int, n_head: c_int, n_kv_head: c_int, head_dim: c_int,
        seq_rows: c_longlong, qkv_stride: c_int, out_stride: c_int,
    ) -> c_int;
    pub fn mx230_attn_decode_partial(
        h: *mut Mx230Handle, stream: *mut c_void, part_m: *mut f32, part_l: *mut f32, part_acc: *mut f32,
        qkv: *const f32, kcache: *const f32, vcache: *const f32, kq: *const i8, vq: *const i8, ks: *const f32,
        vs: *const f32, kb: *const f32, vb: *const f32, t0: c_int, t1: c_int, n_seq: c_int, n_head: c_int,
        n_kv_head: c_int, head_dim: c_int, seq_rows: c_longlong, qkv_stride: c_int,
    ) -> c_int;
    pub fn mx230_merge_partials(
        h: *mut Mx230Handle, stream: *mut c_void, out: *mut f32, m: *const f32, l: *const f32, acc: *const f32,
        parts: c_int, rows: c_int, head_dim: c_int,
    ) -> c_int;
    pub fn mx230_merge_partials_packed(
        h: *mut Mx230Handle, stream: *mut c_void, out: *mut f32, gathered: *const f32, parts: c_int, rows: c_int,
        head_dim: c_int,
    ) -> c_int;
    pub fn mx230_splitkv_comm_create(
        h: *mut Mx230Handle, rank: c_int, world: c_int, rows: c_int, head_dim: c_int,
        out: *mut *mut Mx230SplitKvComm,
    ) -> c_int;
    pub fn mx230_splitkv_comm_export(c: *mut Mx230SplitKvComm, handle64: *mut u8) -> c_int;
    pub fn mx230_splitkv_comm_import(c: *mut Mx230SplitKvComm, peer: c_int, handle64: *const u8) -> c_int;
    pub fn mx230_splitkv_comm_region(c: *mut Mx230SplitKvComm, base: *mut *mut c_void, bytes: *mut usize) -> c_int;
    pub fn mx230_splitkv_comm_attach(c: *mut Mx230SplitKvComm, peer: c_int, region: *mut c_void) -> c_int;
    pub fn mx230_splitkv_exchange_merge(
        c: *mut Mx230SplitKvComm, stream: *mut c_void, out: *mut f32, local: *const f32,
    ) -> c_int;
    pub fn mx230_attn_decode_partial_push(
        h: *mut Mx230Handle, stream: *mut c_void, c: *mut Mx230SplitKvComm, qkv: *const f32, kcache: *const f32,
        vcache: *const f32, kq: *const i8, vq: *const i8, ks: *const f32, vs: *const f32, kb: *const f32,
        vb: *const f32, t0: c_int, t1: c_int, n_seq: c_int, n_head: c_int, n_kv_head: c_int, head_dim: c_int,
        seq_rows: c_longlong, qkv_stride: c_int,
    ) -> c_int;
    pub fn mx230_splitkv_wait_merge(c: *mut Mx230SplitKvComm, stream: *mut c_void, out: *mut f32) -> c_int;
    pub fn mx230_attn_decode_splitkv(
        h: *mut Mx230Handle, stream: *mut c_void, c: *mut Mx230SplitKvComm, out: *mut f32, qkv: *const f32,
        kcache: *const f32, vcache: *const f32, kq: *const i8, vq: *const i8, ks: *const f32, vs: *const f32,
        kb: *const f32, vb: *const f32, t0: c_int, t1: c_int, n_seq: c_int, n_head: c_int, n_kv_head: c_int,
        head_dim: c_int, seq_rows: c_longlong, qkv_stride: c_int,
    ) -> c_int;
    pub fn mx230_splitkv_comm_disconnect(c: *mut Mx230SplitKvComm) -> c_int;
    pub fn mx230_splitkv_comm_destroy(c: *mut Mx230SplitKvComm);
    pub fn mx230_prefill_workspace_bytes(n_tok: c_int, n_keys: c_int, n_head: c_int, n_kv_head: c_int) -> usize;
    pub fn mx230_attn_prefill(
        h: *mut Mx230Handle, stream: *mut c_void, out: *mut f32, qkv: *const f32, kcache: *const f32,
        vcache: *const f32, pos0: c_int, n_tok: c_int, n_head: c_int, n_kv_head: c_int, qkv_stride: c_int,
        out_stride: c_int,
    ) -> c_int;
    pub fn mx230_attn_prefill_paged(
        h: *mut Mx230Handle, stream: *mut c_void, out: *mut f32, qkv: *const f32, kcache: *const f32,
        vcache: *const f32, pos0: c_int, n_tok: c_int, n_head: c_int, n_kv_head: c_int, qkv_stride: c_int,
        out_stride: c_int, bt: *const c_int, bs: c_int,
    ) -> c_int;
    pub fn mx230_attn_prefill_q8(
        h: *mut Mx230Handle, stream: *mut c_void, out: *mut f32, qkv: *const f32, kq: *const i8, vq: *const i8,
        ks: *const f32, vs: *const f32, kb: *const f32, vb: *const f32, pos0: c_int, n_tok: c_int, n_head: c_int,
        n_kv_head: c_int, qkv_stride: c_int, out_stride: c_int,
    ) -> c_int;
    pub fn mx230_attn_prefill_q8_paged(
        h: *mut Mx230Handle, stream: *mut c_void, out: *mut f32, qkv: *const f32, kq: *const i8, vq: *const i8,
        ks: *const f32, vs: *const f32, kb: *const f32, vb: *const f32, pos0: c_int, n_tok: c_int, n_head: c_int,
        n_kv_head: c_int, qkv_stride: c_int, out_stride: c_int, bt: *const c_int, bs: c_int,
    ) -> c_int;
    pub fn mx230_attn_prefill_dp4a(
        h: *mut Mx230Handle, stream: *mut c_void, out: *mut f32, qkv: *const f32, kcache: *const f32,
        vcache: *const f32, pos0: c_int, n_tok: c_int, n_head: c_int, n_kv_head: c_int, qkv_stride: c_int,
        out_stride: c_int,
    ) -> c_int;
    pub fn mx230_attn_prefill_dp4a_paged(
        h: *mut Mx230Handle, stream: *mut c_void, out: *mut f32, qkv: *const f32, kcache: *const f32,
        vcache: *const f32, pos0: c_int, n_tok: c_int, n_head: c_int, n_kv_head: c_int, qkv_stride: c_int,
        out_stride: c_int, bt: *const c_int, bs: c_int,
    ) -> c_int;
    pub fn mx230_gemv(
        h: *mut Mx230Handle, stream: *mut c_void, y: *mut f32, x: *const f32, w: *const c_void, w_fp16: c_int,
        b: *const f32, n_in: c_int, n_out: c_int, accum: c_int,
    ) -> c_int;
    pub fn mx230_gemm_workspace_bytes(m: c_int, n: c_int, k: c_int, w_fp16: c_int) -> usize;
    pub fn mx230_gemm(
        h: *mut Mx230Handle, stream: *mut c_void, C: *mut f32, A: *const f32, w: *const c_void, w_fp16: c_int,
        bias: *const f32, m: c_int, n: c_int, k: c_int,
    ) -> c_int;
    pub fn mx230_gemv_int8(
        h: *mut Mx230Handle, stream: *mut c_void, y: *mut f32, x: *const f32, w_packed: *const c_void,
        scales: *const f32, b: *const f32, n_in: c_int, n_out: c_int, accum: c_int, act_group: c_int,
    ) -> c_int;
    pub fn mx230_qkv_rope_kvwrite(
        h: *mut Mx230Handle, stream: *mut c_void, qkv: *mut f32, x: *const f32, w: *const c_void, w_kind: c_int,
        w_scales: *const f32, act_group: c_int, b: *const f32, n_in: c_int, pos: c_int, pos_ptr: *const c_int,
        n_head: c_int, n_kv_head: c_int, head_dim: c_int, theta: f32, kcache: *mut f32, vcache: *mut f32,
        kq: *mut i8, vq: *mut i8, ks: *mut f32, vs: *mut f32, kb: *mut f32, vb: *mut f32, bt: *const c_int,
        bs: c_int,
    ) -> c_int;
    pub fn mx230_kv_pool_create(
        out: *mut *mut Mx230KvPool, n_slots: c_int, block_size: c_int, prefix_cache: c_int,
    ) -> c_int;
    pub fn mx230_kv_pool_destroy(p: *mut Mx230KvPool);
    pub fn mx230_kv_pool_n_blocks(p: *const Mx230KvPool) -> c_int;
    pub fn mx230_kv_pool_block_size(p: *const Mx230KvPool) -> c_int;
    pub fn mx230_kv_pool_free_blocks(p: *const Mx230KvPool) -> c_int;
    pub fn mx230_kv_pool_cached_blocks(p: *const Mx230KvPool) -> c_int;
    pub fn mx230_kv_pool_evictions(p: *const Mx230KvPool) -> c_longlong;
    pub fn mx230_kv_pool_refcount(p: *const Mx230KvPool, block: c_int) -> c_int;
    pub fn mx230_kv_pool_table(p: *const Mx230KvPool, table_out: *mut c_int, n: c_int) -> c_int;
    pub fn mx230_kv_pool_phys_row(p: *const Mx230KvPool, t: c_int) -> c_int;
    pub fn mx230_kv_pool_alloc(p: *mut Mx230KvPool, block_out: *mut c_int) -> c_int;
    pub fn mx230_kv_pool_incref(p: *mut Mx230KvPool, block: c_int) -> c_int;
    pub fn mx230_kv_pool_decref(p: *mut Mx230KvPool, block: c_int) -> c_int;
    pub fn mx230_kv_pool_evict(p: *mut Mx230KvPool, freed_block: *mut c_int) -> c_int;
    pub fn mx230_kv_pool_lookup(
        p: *mut Mx230KvPool, tokens: *const u32, n: c_int, blocks_out: *mut c_int, cap: c_int,
        n_matched: *mut c_int,
    ) -> c_int;
    pub fn mx230_kv_pool_insert(
        p: *mut Mx230KvPool, tokens: *const u32, n: c_int, blocks: *const c_int, n_blk: c_int,
        created_out: *mut c_int, cap: c_int, n_created: *mut c_int,
    ) -> c_int;
    pub fn mx230_kv_pool_begin_request(
        p: *mut Mx230KvPool, tokens: *const u32, n: c_int, reused_tokens: *mut c_int,
    ) -> c_int;
    pub fn mx230_kv_pool_end_request(p: *mut Mx230KvPool, tokens: *const u32, n: c_int) -> c_int;
    pub fn mx230_kv_pool_abort_request(p: *mut Mx230KvPool) -> c_int;
    pub fn mx230_kv_pool_audit(p: *const Mx230KvPool) -> c_int;
    pub fn mx230_sched_create(
        out: *mut *mut Mx230Sched, pool: *mut Mx230KvPool, n_ctx: c_int, max_batch: c_int, prompt_len: *const c_int,
        max_new: *const c_int, n_requests: c_int,
    ) -> c_int;
    pub fn mx230_sched_destroy(s: *mut Mx230Sched);
    pub fn mx230_sched_n_log(s: *const Mx230Sched) -> c_int;
    pub fn mx230_sched_admit(s: *mut Mx230Sched, request: *mut c_int, table_out: *mut c_int) -> c_int;
    pub fn mx230_sched_admitted(s: *mut Mx230Sched, request: c_int, first_token: u32) -> c_int;
    pub fn mx230_sched_batch(
        s: *mut Mx230Sched, n_active: *mut c_int, cur: *mut u32, pos: *mut c_int, tables: *mut c_int,
    ) -> c_int;
    pub fn mx230_sched_step_done(s: *mut Mx230Sched, next_tokens: *const u32) -> c_int;
    pub fn mx230_sched_result(
        s: *const Mx230Sched, request: c_int, out: *mut u32, cap: c_int, n: *mut c_int,
    ) -> c_int;
    pub fn mx230_sched_stat(s: *const Mx230Sched, which: c_int) -> c_longlong;
}
