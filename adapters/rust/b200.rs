//! B200 backend for LeafcutterLLM: `impl Backend` and `Engine` / `ShardEngine`-shaped wrappers over
//! `libleafcutter_b200.so` (C ABI in `include/leafcutter_b200.h`).
//!
//! NOT COMPILED IN THIS REPOSITORY: the build image has no Rust toolchain.  This is the file a maintainer drops into the
//! reference crate as `rust/src/backend/b200.rs` (add `pub mod b200;` to `rust/src/backend/mod.rs` and
//! `println!("cargo:rustc-link-lib=dylib=leafcutter_b200");` to a `build.rs`).
//!
//! What it replaces, by reference file:line
//!   * `trait Backend` (`rust/src/backend/mod.rs:18-46`) — `B200Backend`, one FFI call per method, same slices in,
//!     a freshly allocated `Vec<f32>` out, panics where the reference asserts (`rust/src/model/tensor.rs:108-113`).
//!   * `Engine::{load, forward, generate}` (`rust/src/inference/engine.rs:18-132`) — `B200Engine`.
//!   * `ShardEngine::{load_with_cache, forward, generate, reset_kv_cache, kv_cache_memory_mb}`
//!     (`rust/src/inference/shard_engine.rs:27-167`) — `B200ShardEngine`.
//!   * `sample_top_p` (`rust/src/inference/sampler.rs:6-50`) — `sample_top_p`, the random draw stays on the Rust side.
//!
//! Install the backend once, as the reference does for its own (`backend/mod.rs:58-60`):
//!     `Tensor::set_global_backend(&backend::b200::B200_BACKEND);`
//! A per-operator backend moves every operand over PCIe per call (as the reference's wgpu backend does,
//! `rust/src/backend/wgpu.rs:158-236`); it is the level for parity, not for speed.  Speed comes from `B200Engine`,
//! which keeps weights, KV cache and activations on the device.

use super::Backend;
use std::ffi::{c_void, CStr, CString};
use std::os::raw::c_char;

#[repr(C)]
#[derive(Clone, Copy, Default)]
pub struct LcModelConfig {
    pub hidden_size: i32,
    pub num_layers: i32,
    pub num_heads: i32,
    pub num_kv_heads: i32,
    pub intermediate_size: i32,
    pub max_seq_len: i32,
    pub vocab_size: i32,
    pub rope_theta: f32,
    pub rms_eps: f32,       // 0 -> 1e-5 (engine.rs:102,111,121)
    pub kv_dtype: i32,      // 0 = f16 as rust/src/cache/mod.rs:33-61
    pub rope_mode: i32,     // 0 = position inside the call, as attention.rs:13-21
    pub n_experts: i32,
    pub top_k: i32,
    pub max_seqs: i32,
    pub kv_page_tokens: i32,
    pub kv_pool_tokens: i64,
    pub device: i32,
    pub tp_size: i32,
    pub tp_rank: i32,
    pub reserved: [i32; 5],
}

#[repr(C)]
pub struct LcModel { _private: [u8; 0] }
#[repr(C)]
pub struct LcShardEngine { _private: [u8; 0] }

extern "C" {
    fn lc_last_error() -> *const c_char;
    fn lc_matmul_f32(a: *const f32, b: *const f32, m: usize, k: usize, n: usize, c: *mut f32) -> i32;
    fn lc_vec_add(a: *const f32, b: *const f32, n: usize, out: *mut f32) -> i32;
    fn lc_vec_mul(a: *const f32, b: *const f32, n: usize, out: *mut f32) -> i32;
    fn lc_vec_scale(a: *const f32, scale: f32, n: usize, out: *mut f32) -> i32;
    fn lc_vec_scale_mul(a: *const f32, scale: f32, b: *const f32, n: usize, out: *mut f32) -> i32;
    fn lc_rms_norm(x: *const f32, w: *const f32, eps: f32, hidden: usize, rows: usize, out: *mut f32) -> i32;
    fn lc_silu(x: *const f32, n: usize, out: *mut f32) -> i32;
    fn lc_softmax(x: *const f32, hidden: usize, rows: usize, out: *mut f32) -> i32;
    fn lc_sum_sq(x: *const f32, n: usize, out: *mut f32) -> i32;
    fn lc_qmatmul(typ: u32, a: *const f32, w_blocks: *const u8, m: usize, k: usize, n: usize, c: *mut f32) -> i32;
    fn lc_q8_0_matmul_shard(a: *const f32, scales: *const f32, qs: *const i8, m: usize, k: usize, n: usize, c: *mut f32) -> i32;
    fn lc_q4_0_matmul_shard(a: *const f32, scales: *const f32, qs: *const u8, m: usize, k: usize, n: usize, c: *mut f32) -> i32;
    fn lc_sample_top_p(logits: *const f32, n: usize, temperature: f32, top_p: f32, u: f32, token: *mut i64) -> i32;

    fn lc_model_create(cfg: *const LcModelConfig, out: *mut *mut LcModel) -> i32;
    fn lc_model_load_gguf(path: *const c_char, overrides: *const LcModelConfig, out: *mut *mut LcModel) -> i32;
    fn lc_model_set_tensor(m: *mut LcModel, name: *const c_char, typ: u32, dims: *const u64, ndims: i32, bytes: *const u8, nbytes: usize) -> i32;
    fn lc_model_finalize(m: *mut LcModel) -> i32;
    fn lc_model_get_config(m: *const LcModel, out: *mut LcModelConfig) -> i32;
    fn lc_model_destroy(m: *mut LcModel) -> i32;
    fn lc_kv_clear(m: *mut LcModel, seq: i32) -> i32;
    fn lc_kv_memory_bytes(m: *const LcModel, out: *mut u64) -> i32;
    fn lc_forward(m: *mut LcModel, tokens: *const i64, n: i32, logits: *mut f32) -> i32;
    fn lc_generate(m: *mut LcModel, tokens: *const i64, n: i32, max_tokens: i32, temperature: f32, top_p: f32, stop_on_eos: i32,
                   out: *mut i64, n_out: *mut i32, cb: Option<extern "C" fn(i64, *mut c_void)>, user: *mut c_void) -> i32;
    fn lc_model_set_seed(m: *mut LcModel, seed: u64) -> i32;

    fn lc_shard_engine_load(manifest_path: *const c_char, max_seq_len: i32, device: i32, out: *mut *mut LcShardEngine) -> i32;
    fn lc_shard_engine_forward(e: *mut LcShardEngine, tokens: *const i64, n: i32, logits: *mut f32, next: *mut i64) -> i32;
    fn lc_shard_engine_generate(e: *mut LcShardEngine, tokens: *const i64, n: i32, max_tokens: i32, temperature: f32, top_p: f32,
                                out: *mut i64, n_out: *mut i32) -> i32;
    fn lc_shard_engine_set_seed(e: *mut LcShardEngine, seed: u64) -> i32;
    fn lc_shard_engine_reset_kv_cache(e: *mut LcShardEngine) -> i32;
    fn lc_shard_engine_kv_cache_memory_bytes(e: *mut LcShardEngine, out: *mut u64) -> i32;
    fn lc_shard_engine_destroy(e: *mut LcShardEngine) -> i32;
}

fn last_error() -> String {
    unsafe { CStr::from_ptr(lc_last_error()) }.to_string_lossy().into_owned()
}

/// The trait is infallible (shape errors are asserts in `Tensor`, tensor.rs:108-113,139): keep that behaviour.
fn must(rc: i32) {
    if rc != 0 {
        panic!("leafcutter_b200: {}", last_error());
    }
}

fn ok(rc: i32) -> Result<(), Box<dyn std::error::Error>> {
    if rc == 0 { Ok(()) } else { Err(last_error().into()) }
}

// ---------------------------------------------------------------------------------------------------------------------
// trait Backend (rust/src/backend/mod.rs:18-46)
// ---------------------------------------------------------------------------------------------------------------------
pub struct B200Backend;
pub static B200_BACKEND: B200Backend = B200Backend;

impl Backend for B200Backend {
    fn matmul(&self, a: &[f32], b: &[f32], m: usize, k: usize, n: usize) -> Vec<f32> {
        assert_eq!(a.len(), m * k);
        assert_eq!(b.len(), k * n);
        let mut c = vec![0.0f32; m * n];
        must(unsafe { lc_matmul_f32(a.as_ptr(), b.as_ptr(), m, k, n, c.as_mut_ptr()) });
        c
    }
    fn vec_add(&self, a: &[f32], b: &[f32]) -> Vec<f32> {
        assert_eq!(a.len(), b.len());
        let mut out = vec![0.0f32; a.len()];
        must(unsafe { lc_vec_add(a.as_ptr(), b.as_ptr(), a.len(), out.as_mut_ptr()) });
        out
    }
    fn vec_mul(&self, a: &[f32], b: &[f32]) -> Vec<f32> {
        assert_eq!(a.len(), b.len());
        let mut out = vec![0.0f32; a.len()];
        must(unsafe { lc_vec_mul(a.as_ptr(), b.as_ptr(), a.len(), out.as_mut_ptr()) });
        out
    }
    fn vec_scale(&self, a: &[f32], scale: f32) -> Vec<f32> {
        let mut out = vec![0.0f32; a.len()];
        must(unsafe { lc_vec_scale(a.as_ptr(), scale, a.len(), out.as_mut_ptr()) });
        out
    }
    fn vec_scale_mul(&self, a: &[f32], scale: f32, b: &[f32]) -> Vec<f32> {
        assert_eq!(a.len(), b.len());
        let mut out = vec![0.0f32; a.len()];
        must(unsafe { lc_vec_scale_mul(a.as_ptr(), scale, b.as_ptr(), a.len(), out.as_mut_ptr()) });
        out
    }
    fn rms_norm(&self, x: &[f32], weight: &[f32], eps: f32, hidden_size: usize) -> Vec<f32> {
        assert_eq!(weight.len(), hidden_size);
        assert_eq!(x.len() % hidden_size, 0);
        let mut out = vec![0.0f32; x.len()];
        must(unsafe { lc_rms_norm(x.as_ptr(), weight.as_ptr(), eps, hidden_size, x.len() / hidden_size, out.as_mut_ptr()) });
        out
    }
    fn silu(&self, x: &[f32]) -> Vec<f32> {
        let mut out = vec![0.0f32; x.len()];
        must(unsafe { lc_silu(x.as_ptr(), x.len(), out.as_mut_ptr()) });
        out
    }
    fn softmax(&self, x: &[f32], hidden_size: usize) -> Vec<f32> {
        assert_eq!(x.len() % hidden_size, 0);
        let mut out = vec![0.0f32; x.len()];
        must(unsafe { lc_softmax(x.as_ptr(), hidden_size, x.len() / hidden_size, out.as_mut_ptr()) });
        out
    }
    fn sum_sq(&self, x: &[f32]) -> f32 {
        let mut out = 0.0f32;
        must(unsafe { lc_sum_sq(x.as_ptr(), x.len(), &mut out) });
        out
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// The quantised-matmul free functions `Tensor::matmul` calls when the right-hand side carries `q_data`
// (rust/src/model/tensor.rs:116-131; rust/src/kernels/int8_gemm.rs:172-194, 336-358).  The reference's matrices keep
// `blocks: Vec<Block>` with an f32 scale and 32 quants per block, laid [k rows][n / 32]; the library takes the scales
// and the quants as two flat arrays in that same order.
// ---------------------------------------------------------------------------------------------------------------------
pub fn q8_0_matmul(a: &[f32], scales: &[f32], qs: &[i8], c: &mut [f32], m: usize, k: usize, n: usize) {
    assert_eq!(a.len(), m * k);
    assert_eq!(qs.len(), k * n);
    assert_eq!(scales.len(), k * n / 32);
    assert_eq!(c.len(), m * n);
    must(unsafe { lc_q8_0_matmul_shard(a.as_ptr(), scales.as_ptr(), qs.as_ptr(), m, k, n, c.as_mut_ptr()) });
}
pub fn q4_0_matmul(a: &[f32], scales: &[f32], qs: &[u8], c: &mut [f32], m: usize, k: usize, n: usize) {
    assert_eq!(a.len(), m * k);
    assert_eq!(qs.len(), k * n / 2);
    assert_eq!(scales.len(), k * n / 32);
    assert_eq!(c.len(), m * n);
    must(unsafe { lc_q4_0_matmul_shard(a.as_ptr(), scales.as_ptr(), qs.as_ptr(), m, k, n, c.as_mut_ptr()) });
}
/// `c[m, n] = a[m, k] . dequant(W)^T` straight from the raw GGUF blocks `GGUFile::get_tensor_raw` returns
/// (rust/src/model/gguf.rs:121-127): no dequantise, no transpose (what rust/src/model/loader.rs:145-168 would do first).
pub fn gguf_qmatmul(ggml_type: u32, a: &[f32], raw_blocks: &[u8], m: usize, k: usize, n: usize) -> Vec<f32> {
    assert_eq!(a.len(), m * k);
    let mut c = vec![0.0f32; m * n];
    must(unsafe { lc_qmatmul(ggml_type, a.as_ptr(), raw_blocks.as_ptr(), m, k, n, c.as_mut_ptr()) });
    c
}

/// `sample_top_p` (rust/src/inference/sampler.rs:6-50): the draw `u` is the caller's `rng.gen::<f32>()` (:38-39), so the
/// token is the one the CPU code would have picked for that draw; `temperature <= 0` is the greedy branch (:7-10).
pub fn sample_top_p(logits: &[f32], temperature: f32, top_p: f32, u: f32) -> usize {
    assert!(!logits.is_empty());
    let mut tok = 0i64;
    must(unsafe { lc_sample_top_p(logits.as_ptr(), logits.len(), temperature, top_p, u, &mut tok) });
    tok as usize
}

// ---------------------------------------------------------------------------------------------------------------------
// Engine (rust/src/inference/engine.rs)
// ---------------------------------------------------------------------------------------------------------------------
pub struct B200Engine {
    handle: *mut LcModel,
    pub config: LcModelConfig,
}
// The reference serialises its engine with Arc<Mutex<Engine>> (rust/src/api/mod.rs:42,50); one handle must be used the same way.
unsafe impl Send for B200Engine {}

extern "C" fn token_trampoline(tok: i64, user: *mut c_void) {
    let f = unsafe { &mut *(user as *mut &mut dyn FnMut(usize)) };
    f(tok as usize);
}

impl B200Engine {
    /// `Engine::load(path)` (engine.rs:18-49): the library parses the GGUF v3 container itself (header, config keys and
    /// their fallbacks as rust/src/model/gguf.rs:76-119 and loader.rs:106-133) and uploads the raw blocks.
    pub fn load(path: &str) -> Result<Self, Box<dyn std::error::Error>> {
        let c_path = CString::new(path)?;
        let mut h: *mut LcModel = std::ptr::null_mut();
        ok(unsafe { lc_model_load_gguf(c_path.as_ptr(), std::ptr::null(), &mut h) })?;
        let mut config = LcModelConfig::default();
        ok(unsafe { lc_model_get_config(h, &mut config) })?;
        Ok(Self { handle: h, config })
    }

    /// The same for a crate that keeps its own parser and capability report: create, hand over every tensor as the raw
    /// bytes of `get_tensor_raw` with its GGUF name, dims (fastest first) and type code, finalize.
    pub fn from_tensors<'a, I>(config: LcModelConfig, tensors: I) -> Result<Self, Box<dyn std::error::Error>>
    where
        I: IntoIterator<Item = (&'a str, u32, &'a [u64], &'a [u8])>,
    {
        let mut h: *mut LcModel = std::ptr::null_mut();
        ok(unsafe { lc_model_create(&config, &mut h) })?;
        let engine = Self { handle: h, config };
        for (name, typ, dims, raw) in tensors {
            let c_name = CString::new(name)?;
            ok(unsafe { lc_model_set_tensor(h, c_name.as_ptr(), typ, dims.as_ptr(), dims.len() as i32, raw.as_ptr(), raw.len()) })?;
        }
        ok(unsafe { lc_model_finalize(h) })?;
        Ok(engine)
    }

    /// `Engine::forward(&tokens)` (engine.rs:78-132): appends to the KV cache, returns the logits of the last token.
    pub fn forward(&mut self, tokens: &[usize]) -> Vec<f32> {
        let toks: Vec<i64> = tokens.iter().map(|&t| t as i64).collect();
        let mut logits = vec![0.0f32; self.config.vocab_size as usize];
        must(unsafe { lc_forward(self.handle, toks.as_ptr(), toks.len() as i32, logits.as_mut_ptr()) });
        logits
    }

    /// `Engine::generate` (engine.rs:51-76): clears the cache, first token from the prefill, stops after token id 2.
    /// `temperature > 0` needs `set_seed` first (the reference draws from an unseeded generator, sampler.rs:38-39).
    pub fn generate(&mut self, tokens: &[usize], max_tokens: usize, temperature: f32, top_p: f32) -> Vec<usize> {
        self.generate_with(tokens, max_tokens, temperature, top_p, None)
    }

    pub fn generate_with(&mut self, tokens: &[usize], max_tokens: usize, temperature: f32, top_p: f32,
                         on_token: Option<&mut dyn FnMut(usize)>) -> Vec<usize> {
        let toks: Vec<i64> = tokens.iter().map(|&t| t as i64).collect();
        let mut out = vec![0i64; max_tokens];
        let mut n_out = 0i32;
        let rc = match on_token {
            Some(mut f) => {
                let user = &mut f as *mut &mut dyn FnMut(usize) as *mut c_void;
                unsafe { lc_generate(self.handle, toks.as_ptr(), toks.len() as i32, max_tokens as i32, temperature, top_p, 1,
                                     out.as_mut_ptr(), &mut n_out, Some(token_trampoline), user) }
            }
            None => unsafe { lc_generate(self.handle, toks.as_ptr(), toks.len() as i32, max_tokens as i32, temperature, top_p, 1,
                                         out.as_mut_ptr(), &mut n_out, None, std::ptr::null_mut()) },
        };
        must(rc);
        out[..n_out as usize].iter().map(|&t| t as usize).collect()
    }

    pub fn set_seed(&mut self, seed: u64) { must(unsafe { lc_model_set_seed(self.handle, seed) }); }
    /// `KVCache::clear` (rust/src/cache/mod.rs:26-30)
    pub fn clear_cache(&mut self) { must(unsafe { lc_kv_clear(self.handle, -1) }); }
    /// `KVCache::memory_bytes` (rust/src/cache/mod.rs:80-84)
    pub fn kv_memory_bytes(&self) -> u64 {
        let mut v = 0u64;
        must(unsafe { lc_kv_memory_bytes(self.handle, &mut v) });
        v
    }
}

impl Drop for B200Engine {
    fn drop(&mut self) {
        unsafe { lc_model_destroy(self.handle) };
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// ShardEngine (rust/src/inference/shard_engine.rs)
// ---------------------------------------------------------------------------------------------------------------------
pub struct B200ShardEngine {
    handle: *mut LcShardEngine,
    vocab_size: usize,
}
unsafe impl Send for B200ShardEngine {}

impl B200ShardEngine {
    /// `ShardEngine::load_with_cache(manifest_path, num_layers)` (:34-61): every layer stays in device memory, so the
    /// number of cache slots is moot.  `vocab_size` is the manifest's (rust/src/shard/loader.rs:13-50).
    pub fn load_with_cache(manifest_path: &str, _cache_slots: usize, vocab_size: usize) -> Result<Self, Box<dyn std::error::Error>> {
        let c_path = CString::new(manifest_path)?;
        let mut h: *mut LcShardEngine = std::ptr::null_mut();
        ok(unsafe { lc_shard_engine_load(c_path.as_ptr(), 0, 0, &mut h) })?;
        Ok(Self { handle: h, vocab_size })
    }
    /// `ShardEngine::forward` (:99-167)
    pub fn forward(&mut self, tokens: &[usize]) -> Vec<f32> {
        let toks: Vec<i64> = tokens.iter().map(|&t| t as i64).collect();
        let mut logits = vec![0.0f32; self.vocab_size];
        must(unsafe { lc_shard_engine_forward(self.handle, toks.as_ptr(), toks.len() as i32, logits.as_mut_ptr(), std::ptr::null_mut()) });
        logits
    }
    /// `ShardEngine::generate` (:74-97)
    pub fn generate(&mut self, tokens: &[usize], max_tokens: usize, temperature: f32, top_p: f32) -> Vec<usize> {
        let toks: Vec<i64> = tokens.iter().map(|&t| t as i64).collect();
        let mut out = vec![0i64; max_tokens];
        let mut n_out = 0i32;
        must(unsafe { lc_shard_engine_generate(self.handle, toks.as_ptr(), toks.len() as i32, max_tokens as i32, temperature, top_p,
                                               out.as_mut_ptr(), &mut n_out) });
        out[..n_out as usize].iter().map(|&t| t as usize).collect()
    }
    pub fn set_seed(&mut self, seed: u64) { must(unsafe { lc_shard_engine_set_seed(self.handle, seed) }); }
    /// `reset_kv_cache` (:64-66)
    pub fn reset_kv_cache(&mut self) { must(unsafe { lc_shard_engine_reset_kv_cache(self.handle) }); }
    /// `kv_cache_memory_mb` (:69-71)
    pub fn kv_cache_memory_mb(&mut self) -> f64 {
        let mut v = 0u64;
        must(unsafe { lc_shard_engine_kv_cache_memory_bytes(self.handle, &mut v) });
        v as f64 / (1024.0 * 1024.0)
    }
}

impl Drop for B200ShardEngine {
    fn drop(&mut self) {
        unsafe { lc_shard_engine_destroy(self.handle) };
    }
}
