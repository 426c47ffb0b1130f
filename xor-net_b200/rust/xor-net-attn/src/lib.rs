//! Drop-in for `xor_net::nn::{fast_attention, CpuRingCache}` backed by the B200 attention library.
//! NOT BUILT in this repository's environment (no Rust toolchain there).
//!
//! `fast_attention` keeps the signature of src/nn/fast_attention.rs:75-85; `DeviceKvCache` stands
//! where `CpuRingCache` (src/nn/fast_attention.rs:18-60) stood and keeps its constructor.
use std::os::raw::{c_char, c_void};
use std::sync::{Arc, Mutex, OnceLock, Weak};
use std::collections::HashMap;

#[repr(C)] pub struct XnCtx { _p: [u8; 0] }
#[repr(C)] pub struct XnStream { _p: [u8; 0] }

#[repr(C)]
pub struct XnCtxDesc {
    pub device: i32, pub num_layers: i32, pub num_heads: i32, pub num_kv_heads: i32,
    pub head_dim: i32, pub page_tokens: i32, pub pool_pages: i64, pub pool_bytes: i64,
    pub shuffle_seed: u64, pub max_pos: i32, pub prefill_mode: i32,
    pub rope_cos: *const f32, pub rope_sin: *const f32, pub cuda_stream: *mut c_void,
    pub batch_window_us: i32, pub kv_format: i32,
}

/// `XnCtxDesc::kv_format`: the f32 cache `fast_attention` reads, or only the u8 shadow of
/// `CpuRingCache::new(.., use_u8 = true)` (src/nn/fast_attention.rs:42-50) as the cache itself.
pub const XN_KV_F32: i32 = 0;
pub const XN_KV_U8: i32 = 1;

extern "C" {
    fn xn_ctx_create(d: *const XnCtxDesc, out: *mut *mut XnCtx) -> i32;
    fn xn_ctx_destroy(c: *mut XnCtx) -> i32;
    fn xn_stream_create(c: *mut XnCtx, max_seq_len: i64, out: *mut *mut XnStream) -> i32;
    fn xn_stream_destroy(c: *mut XnCtx, s: *mut XnStream) -> i32;
    fn xn_attention(c: *mut XnCtx, s: *mut XnStream, layer: i32, index_pos: i64, seq_len: i32,
                    q: *const f32, k: *const f32, v: *const f32, out: *mut f32) -> i32;
    fn xn_kv_read_range(c: *mut XnCtx, s: *mut XnStream, layer: i32, t0: i64, n: i64,
                        k: *mut f32, v: *mut f32) -> i32;
    fn xn_last_error(c: *mut XnCtx) -> *const c_char;
    // the projections around the attention (models/llama/attention.rs:52-89 and :103-108)
    fn xn_qkv_proj_set(c: *mut XnCtx, d: *const XnQkvProjDesc) -> i32;
    fn xn_out_proj_set(c: *mut XnCtx, d: *const XnOutProjDesc) -> i32;
    fn xn_attention_batch(c: *mut XnCtx, n: i32, reqs: *const XnReq) -> i32;
}

/// Request flags of `xn_req.flags` (include/xn_attn.h).
pub const XN_REQ_OUT_PROJ: u32 = 1 << 4;
pub const XN_REQ_QKV_PROJ: u32 = 1 << 5;

#[repr(C)]
pub struct XnReq {
    pub stream: *mut XnStream, pub layer: i32, pub seq_len: i32, pub index_pos: i64,
    pub q: *const f32, pub k: *const f32, pub v: *const f32, pub out: *mut f32,
    pub flags: u32, pub reserved: u32,
}

/// `xn_qkv_proj_desc`: the dense `TernaryLinear`s q_proj / k_proj / v_proj of one layer.
#[repr(C)]
pub struct XnQkvProjDesc {
    pub layer: i32, pub in_dim: i32, pub pack_type: i32, pub reserved: i32,
    pub q_packed: *const u8, pub q_scales: *const f32,
    pub k_packed: *const u8, pub k_scales: *const f32,
    pub v_packed: *const u8, pub v_scales: *const f32,
}

/// `xn_out_proj_desc`: o_proj (dense `TernaryLinear`) and the optional sub-norm of one layer.
#[repr(C)]
pub struct XnOutProjDesc {
    pub layer: i32, pub in_dim: i32, pub out_dim: i32, pub pack_type: i32,
    pub packed: *const u8, pub w_scales: *const f32, pub norm_weight: *const f32,
    pub norm_eps: f32, pub reserved: u32,
}

/// The tensor type of the reference (src/tensor.rs:6-10), re-declared so the crate stands alone;
/// inside xor-net use `xor_net::tensor::FastTensor` instead.
#[derive(Clone, Debug)]
pub struct FastTensor { pub data: Vec<f32>, pub shape: Vec<usize> }
impl FastTensor { pub fn new(data: Vec<f32>, shape: Vec<usize>) -> Self { Self { data, shape } } }

/// One page pool per (device, model shape), shared like the `Arc<Llama>` of server/main.rs:613-645.
pub struct AttnContext(*mut XnCtx);
unsafe impl Send for AttnContext {}
unsafe impl Sync for AttnContext {}
impl Drop for AttnContext { fn drop(&mut self) { unsafe { xn_ctx_destroy(self.0); } } }

type Key = (i32, usize, usize, usize, usize);
fn registry() -> &'static Mutex<HashMap<Key, Weak<AttnContext>>> {
    static R: OnceLock<Mutex<HashMap<Key, Weak<AttnContext>>>> = OnceLock::new();
    R.get_or_init(|| Mutex::new(HashMap::new()))
}

fn shared_context(device: i32, layers: usize, heads: usize, kv_heads: usize, dim: usize,
                  max_seq_len: usize) -> anyhow::Result<Arc<AttnContext>> {
    let mut reg = registry().lock().unwrap();
    let key = (device, layers, heads, kv_heads, dim);
    if let Some(c) = reg.get(&key).and_then(|w| w.upgrade()) { return Ok(c); }
    let pages = std::env::var("XORNET_ATTN_POOL_PAGES").ok().and_then(|s| s.parse::<i64>().ok())
        .unwrap_or((((max_seq_len + 63) / 64) * 64) as i64);
    let desc = XnCtxDesc { device, num_layers: layers as i32, num_heads: heads as i32,
        num_kv_heads: kv_heads as i32, head_dim: dim as i32, page_tokens: 64, pool_pages: pages,
        pool_bytes: 0, shuffle_seed: 0, max_pos: 0, prefill_mode: 0, rope_cos: std::ptr::null(),
        rope_sin: std::ptr::null(), cuda_stream: std::ptr::null_mut(), batch_window_us: 0, kv_format: XN_KV_F32 };
    let mut raw: *mut XnCtx = std::ptr::null_mut();
    let rc = unsafe { xn_ctx_create(&desc, &mut raw) };
    if rc != 0 {
        let msg = unsafe { std::ffi::CStr::from_ptr(xn_last_error(std::ptr::null_mut())) }.to_string_lossy();
        anyhow::bail!("xn_ctx_create failed ({}): {}", rc, msg);
    }
    let c = Arc::new(AttnContext(raw));
    reg.insert(key, Arc::downgrade(&c));
    Ok(c)
}

pub struct DeviceKvCache {
    pub max_seq_len: usize, pub num_kv_heads: usize, pub head_dim: usize,
    num_layers: usize, bound: Option<(Arc<AttnContext>, *mut XnStream)>,
}
unsafe impl Send for DeviceKvCache {}

impl DeviceKvCache {
    /// `CpuRingCache::new` (fast_attention.rs:31-34); `use_u8` is ignored: the reference's u8
    /// shadow is never read.
    pub fn new(num_layers: usize, num_kv_heads: usize, max_seq_len: usize, head_dim: usize, _use_u8: bool) -> Self {
        Self { max_seq_len, num_kv_heads, head_dim, num_layers, bound: None }
    }
    fn bind(&mut self, num_heads: usize) -> anyhow::Result<(*mut XnCtx, *mut XnStream)> {
        if self.bound.is_none() {
            let ctx = shared_context(0, self.num_layers, num_heads, self.num_kv_heads, self.head_dim, self.max_seq_len)?;
            let mut s: *mut XnStream = std::ptr::null_mut();
            let rc = unsafe { xn_stream_create(ctx.0, self.max_seq_len as i64, &mut s) };
            if rc != 0 { anyhow::bail!("xn_stream_create failed ({})", rc); }
            self.bound = Some((ctx, s));
        }
        let (c, s) = self.bound.as_ref().unwrap();
        Ok((c.0, *s))
    }
    /// The reference's pub field `k_buffers[layer]` (index `h*cap*D + t*D + d`), read back.
    pub fn k_buffer(&self, layer: usize) -> Vec<f32> { self.read(layer, true) }
    pub fn v_buffer(&self, layer: usize) -> Vec<f32> { self.read(layer, false) }
    fn read(&self, layer: usize, keys: bool) -> Vec<f32> {
        let mut out = vec![0.0f32; self.num_kv_heads * self.max_seq_len * self.head_dim];
        if let Some((c, s)) = &self.bound {
            let p = out.as_mut_ptr();
            unsafe { xn_kv_read_range(c.0, *s, layer as i32, 0, self.max_seq_len as i64,
                                      if keys { p } else { std::ptr::null_mut() },
                                      if keys { std::ptr::null_mut() } else { p }); }
        }
        out
    }
}
impl Drop for DeviceKvCache {
    fn drop(&mut self) { if let Some((c, s)) = self.bound.take() { unsafe { xn_stream_destroy(c.0, s); } } }
}

/// Same signature as src/nn/fast_attention.rs:75-85 with the cache type swapped.
#[allow(clippy::too_many_arguments)]
pub fn fast_attention(q: &FastTensor, k: &FastTensor, v: &FastTensor, layer_idx: usize,
                      index_pos: usize, cache: &mut DeviceKvCache, num_heads: usize,
                      _num_kv_heads: usize, head_dim: usize) -> anyhow::Result<FastTensor> {
    let (b_sz, seq_len) = match q.shape.as_slice() {
        &[b, _, s, _] => (b, s),
        _ => anyhow::bail!("fast_attention: Q shape must be 4D"),
    };
    if b_sz != 1 {
        anyhow::bail!("fast_attention currently only supports batch size 1, got {}", b_sz);
    }
    let (ctx, stream) = cache.bind(num_heads)?;
    let mut out = vec![0.0f32; num_heads * seq_len * head_dim];
    let rc = unsafe { xn_attention(ctx, stream, layer_idx as i32, index_pos as i64, seq_len as i32,
                                   q.data.as_ptr(), k.data.as_ptr(), v.data.as_ptr(), out.as_mut_ptr()) };
    if rc != 0 {
        let msg = unsafe { std::ffi::CStr::from_ptr(xn_last_error(ctx)) }.to_string_lossy();
        anyhow::bail!("xn_attention failed ({}): {}", rc, msg);
    }
    Ok(FastTensor::new(out, vec![b_sz, num_heads, seq_len, head_dim]))
}
