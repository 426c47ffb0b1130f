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
#[repr(C)] pub struct XnGroup { _p: [u8; 0] }

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
    fn xn_attention_rope(c: *mut XnCtx, s: *mut XnStream, layer: i32, index_pos: i64, seq_len: i32,
                         q: *const f32, k: *const f32, v: *const f32, out: *mut f32) -> i32;
    fn xn_stream_reset(c: *mut XnCtx, s: *mut XnStream) -> i32;
    fn xn_stream_len(c: *mut XnCtx, s: *mut XnStream, layer: i32) -> i64;
    fn xn_stats_get(c: *mut XnCtx, out: *mut XnStats) -> i32;
    fn xn_ctx_synchronize(c: *mut XnCtx) -> i32;
    fn xn_debug_check_guards(c: *mut XnCtx) -> i32;
    // every GPU of the box behind one process: one context per device, a stream lives on one
    fn xn_group_create(d: *const XnCtxDesc, devices: *const i32, n_devices: i32, out: *mut *mut XnGroup) -> i32;
    fn xn_group_destroy(g: *mut XnGroup) -> i32;
    fn xn_group_size(g: *mut XnGroup) -> i32;
    fn xn_group_ctx(g: *mut XnGroup, i: i32) -> *mut XnCtx;
    fn xn_group_stream_create(g: *mut XnGroup, max_seq_len: i64, expected_tokens: i64, policy: i32,
                              ctx_out: *mut *mut XnCtx, out: *mut *mut XnStream) -> i32;
    pub fn xn_place_stream(n_devices: i32, tokens: *const i64, live_streams: *const i64, ticket: u64,
                           policy: i32) -> i32;
    // the projections around the attention (models/llama/attention.rs:52-89 and :103-108)
    fn xn_qkv_proj_set(c: *mut XnCtx, d: *const XnQkvProjDesc) -> i32;
    fn xn_out_proj_set(c: *mut XnCtx, d: *const XnOutProjDesc) -> i32;
    fn xn_attention_batch(c: *mut XnCtx, n: i32, reqs: *const XnReq) -> i32;
}

/// `policy` of `xn_group_stream_create` / `xn_place_stream`.
pub const XN_PLACE_LEAST_LOADED: i32 = 0;
pub const XN_PLACE_ROUND_ROBIN: i32 = 1;

/// `xn_stats` (include/xn_attn.h), counters of one device's context.
#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct XnStats {
    pub calls: u64, pub batches: u64, pub kernel_launches: u64, pub decode_launches: u64,
    pub prefill_launches: u64, pub h2d_bytes: u64, pub d2h_bytes: u64, pub pages_total: u64,
    pub pages_in_use: u64, pub streams_live: u64, pub device_wait_errors: u64, pub coalesced_max: u64,
    pub out_proj_rows: u64, pub plan_reuses: u64, pub out_transfers: u64,
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

/// One group per model shape, shared like the `Arc<Llama>` of server/main.rs:613-645: a context
/// (page pool, queue of concurrent callers) on every GPU that XORNET_ATTN_DEVICES names, or on
/// every visible GPU.  The pool of each device comes from a byte budget, never from a sequence
/// length: XORNET_ATTN_POOL_PAGES pages, else XORNET_ATTN_POOL_MB megabytes, else (both zero in
/// the descriptor) the library takes half of the device's free memory.  Pages leave the pool only
/// as positions are written, so a cache of any `max_seq_len` fits until the tokens actually held
/// exhaust the budget; that call then fails with "out of pages" and changes nothing.
pub struct AttnGroup(*mut XnGroup);
unsafe impl Send for AttnGroup {}
unsafe impl Sync for AttnGroup {}
impl Drop for AttnGroup { fn drop(&mut self) { unsafe { xn_group_destroy(self.0); } } }

impl AttnGroup {
    pub fn devices(&self) -> usize { unsafe { xn_group_size(self.0) }.max(0) as usize }
    /// Counters of the i-th device.
    pub fn stats(&self, i: usize) -> Option<XnStats> {
        let c = unsafe { xn_group_ctx(self.0, i as i32) };
        if c.is_null() { return None; }
        let mut st = XnStats::default();
        if unsafe { xn_stats_get(c, &mut st) } == 0 { Some(st) } else { None }
    }
    /// Waits for all devices; an error of a bounded device-side wait surfaces here.
    pub fn synchronize(&self) -> anyhow::Result<()> {
        for i in 0..self.devices() {
            let c = unsafe { xn_group_ctx(self.0, i as i32) };
            let rc = unsafe { xn_ctx_synchronize(c) };
            if rc != 0 { anyhow::bail!("xn_ctx_synchronize failed on device slot {} ({})", i, rc); }
        }
        Ok(())
    }
    /// Debug aid: checks the guard bytes around every device buffer of every context.
    pub fn check_guards(&self) -> anyhow::Result<()> {
        for i in 0..self.devices() {
            let c = unsafe { xn_group_ctx(self.0, i as i32) };
            if unsafe { xn_debug_check_guards(c) } != 0 {
                let msg = unsafe { std::ffi::CStr::from_ptr(xn_last_error(c)) }.to_string_lossy();
                anyhow::bail!("guard bytes damaged: {}", msg);
            }
        }
        Ok(())
    }
}

type Key = (usize, usize, usize, usize);
fn registry() -> &'static Mutex<HashMap<Key, Weak<AttnGroup>>> {
    static R: OnceLock<Mutex<HashMap<Key, Weak<AttnGroup>>>> = OnceLock::new();
    R.get_or_init(|| Mutex::new(HashMap::new()))
}

fn env_i64(name: &str) -> i64 { std::env::var(name).ok().and_then(|s| s.parse::<i64>().ok()).unwrap_or(0) }

/// The key holds the model shape only.  No sequence length enters the pool's size, so a later,
/// longer cache is served from the same pool on the same terms as the first.
pub fn shared_group(layers: usize, heads: usize, kv_heads: usize, dim: usize) -> anyhow::Result<Arc<AttnGroup>> {
    let mut reg = registry().lock().unwrap();
    let key = (layers, heads, kv_heads, dim);
    if let Some(g) = reg.get(&key).and_then(|w| w.upgrade()) { return Ok(g); }
    let desc = XnCtxDesc { device: 0 /* ignored by a group */, num_layers: layers as i32, num_heads: heads as i32,
        num_kv_heads: kv_heads as i32, head_dim: dim as i32, page_tokens: 64,
        pool_pages: env_i64("XORNET_ATTN_POOL_PAGES"), pool_bytes: env_i64("XORNET_ATTN_POOL_MB") << 20,
        shuffle_seed: 0, max_pos: 0, prefill_mode: 0, rope_cos: std::ptr::null(),
        rope_sin: std::ptr::null(), cuda_stream: std::ptr::null_mut(),
        batch_window_us: env_i64("XORNET_ATTN_BATCH_WINDOW_US") as i32, kv_format: XN_KV_F32 };
    let mut raw: *mut XnGroup = std::ptr::null_mut();
    // n_devices = 0: XORNET_ATTN_DEVICES ("0,1,5") or every visible device
    let rc = unsafe { xn_group_create(&desc, std::ptr::null(), 0, &mut raw) };
    if rc != 0 {
        let msg = unsafe { std::ffi::CStr::from_ptr(xn_last_error(std::ptr::null_mut())) }.to_string_lossy();
        anyhow::bail!("xn_group_create failed ({}): {}", rc, msg);
    }
    let g = Arc::new(AttnGroup(raw));
    reg.insert(key, Arc::downgrade(&g));
    Ok(g)
}

/// Stands where `CpuRingCache` stood.  Deliberately NOT `Clone` (the reference's `Cache` derives
/// it, models/llama/mod.rs:202): a value names pages of one device's pool, and a copy would need a
/// device-side duplicate of every page it holds.  Nothing on the serving path clones a cache
/// (server/main.rs:92 and examples/batch_bench.rs:188 build one per slot / per worker).
pub struct DeviceKvCache {
    pub max_seq_len: usize, pub num_kv_heads: usize, pub head_dim: usize,
    num_layers: usize, expected_tokens: usize,
    bound: Option<(Arc<AttnGroup>, *mut XnCtx, *mut XnStream)>,
}
unsafe impl Send for DeviceKvCache {}

impl DeviceKvCache {
    /// `CpuRingCache::new` (fast_attention.rs:31-34); `use_u8` is ignored: the reference's u8
    /// shadow is never read.
    pub fn new(num_layers: usize, num_kv_heads: usize, max_seq_len: usize, head_dim: usize, _use_u8: bool) -> Self {
        Self { max_seq_len, num_kv_heads, head_dim, num_layers, expected_tokens: 0, bound: None }
    }
    /// Announces how many tokens this cache is going to hold, so that caches created before they
    /// are filled still spread over the GPUs by load.  Call before the first `fast_attention`.
    pub fn with_expected_tokens(mut self, tokens: usize) -> Self { self.expected_tokens = tokens; self }
    /// Binds on first use (the query head count arrives with the first call).  The cache lands on
    /// the GPU that holds the fewest cached or announced tokens (XORNET_ATTN_PLACEMENT=rr: cache
    /// number modulo the number of GPUs) and stays there.
    fn bind(&mut self, num_heads: usize) -> anyhow::Result<(*mut XnCtx, *mut XnStream)> {
        if self.bound.is_none() {
            let group = shared_group(self.num_layers, num_heads, self.num_kv_heads, self.head_dim)?;
            let policy = match std::env::var("XORNET_ATTN_PLACEMENT").as_deref() {
                Ok("rr") | Ok("round_robin") => XN_PLACE_ROUND_ROBIN,
                _ => XN_PLACE_LEAST_LOADED,
            };
            let mut c: *mut XnCtx = std::ptr::null_mut();
            let mut s: *mut XnStream = std::ptr::null_mut();
            let rc = unsafe { xn_group_stream_create(group.0, self.max_seq_len as i64, self.expected_tokens as i64,
                                                     policy, &mut c, &mut s) };
            if rc != 0 {
                let msg = unsafe { std::ffi::CStr::from_ptr(xn_last_error(std::ptr::null_mut())) }.to_string_lossy();
                anyhow::bail!("xn_group_stream_create failed ({}): {}", rc, msg);
            }
            self.bound = Some((group, c, s));
        }
        let (_, c, s) = self.bound.as_ref().unwrap();
        Ok((*c, *s))
    }
    /// A fresh `Cache::new` on the same device: forgets the tokens and returns the pages.
    pub fn reset(&mut self) {
        if let Some((_, c, s)) = &self.bound { unsafe { xn_stream_reset(*c, *s); } }
    }
    /// Tokens held for `layer` (the reference keeps no such counter: it derives it from index_pos).
    pub fn len(&self, layer: usize) -> usize {
        match &self.bound { Some((_, c, s)) => unsafe { xn_stream_len(*c, *s, layer as i32) }.max(0) as usize, None => 0 }
    }
    /// The reference's pub field `k_buffers[layer]` (index `h*cap*D + t*D + d`), read back.
    pub fn k_buffer(&self, layer: usize) -> Vec<f32> { self.read(layer, true) }
    pub fn v_buffer(&self, layer: usize) -> Vec<f32> { self.read(layer, false) }
    fn read(&self, layer: usize, keys: bool) -> Vec<f32> {
        let mut out = vec![0.0f32; self.num_kv_heads * self.max_seq_len * self.head_dim];
        if let Some((_, c, s)) = &self.bound {
            let p = out.as_mut_ptr();
            unsafe { xn_kv_read_range(*c, *s, layer as i32, 0, self.max_seq_len as i64,
                                      if keys { p } else { std::ptr::null_mut() },
                                      if keys { std::ptr::null_mut() } else { p }); }
        }
        out
    }
}
impl Drop for DeviceKvCache {
    fn drop(&mut self) { if let Some((_g, c, s)) = self.bound.take() { unsafe { xn_stream_destroy(c, s); } } }
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

/// `fast_attention` on queries and keys that are NOT yet rotated: the library applies the rotary
/// embedding of models/llama/attention.rs:93-95 (tables given at context creation) on the device.
#[allow(clippy::too_many_arguments)]
pub fn fast_attention_rope(q: &FastTensor, k: &FastTensor, v: &FastTensor, layer_idx: usize,
                           index_pos: usize, cache: &mut DeviceKvCache, num_heads: usize,
                           head_dim: usize) -> anyhow::Result<FastTensor> {
    let (b_sz, seq_len) = match q.shape.as_slice() {
        &[b, _, s, _] => (b, s),
        _ => anyhow::bail!("fast_attention: Q shape must be 4D"),
    };
    if b_sz != 1 {
        anyhow::bail!("fast_attention currently only supports batch size 1, got {}", b_sz);
    }
    let (ctx, stream) = cache.bind(num_heads)?;
    let mut out = vec![0.0f32; num_heads * seq_len * head_dim];
    let rc = unsafe { xn_attention_rope(ctx, stream, layer_idx as i32, index_pos as i64, seq_len as i32,
                                        q.data.as_ptr(), k.data.as_ptr(), v.data.as_ptr(), out.as_mut_ptr()) };
    if rc != 0 {
        let msg = unsafe { std::ffi::CStr::from_ptr(xn_last_error(ctx)) }.to_string_lossy();
        anyhow::bail!("xn_attention_rope failed ({}): {}", rc, msg);
    }
    Ok(FastTensor::new(out, vec![b_sz, num_heads, seq_len, head_dim]))
}
