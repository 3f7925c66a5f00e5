//! Safe Rust surface over `swb200_contracts.h`: a runtime catalog, text-LLM load / generate / stream, snapshot
//! preparation and media generator load / generate, so that consumers written against a `runtime_cuda`-style crate
//! (`catalog()`, `text().load_for_model(..)`, `generate(req, on_event)`) can link this one instead.
//! Structured values cross the boundary as JSON (`serde_json::Value`); pixels come back as `Vec<u8>` RGB8.

use std::ffi::{c_char, c_int, c_longlong, c_void, CStr, CString};
use std::ptr;

use serde_json::Value;

#[repr(C)]
struct RawRuntime {
    _private: [u8; 0],
}

type EventCb = Option<unsafe extern "C" fn(*const c_char, *mut c_void) -> c_int>;

extern "C" {
    fn swb_rt_open(bundle: *const c_char, package_root: *const c_char, out: *mut *mut RawRuntime) -> c_int;
    fn swb_rt_close(rt: *mut RawRuntime);
    fn swb_rt_last_error() -> *const c_char;
    fn swb_rt_free_string(s: *mut c_char);
    fn swb_rt_catalog_json(rt: *mut RawRuntime, out: *mut *mut c_char) -> c_int;
    fn swb_text_load(rt: *mut RawRuntime, provider_id: *const c_char, spec: *const c_char, out: *mut u64) -> c_int;
    fn swb_text_descriptor_json(rt: *mut RawRuntime, handle: u64, out: *mut *mut c_char) -> c_int;
    fn swb_text_generate(rt: *mut RawRuntime, handle: u64, request: *const c_char, cb: EventCb, user: *mut c_void,
                         out: *mut *mut c_char) -> c_int;
    fn swb_prepare_snapshot(rt: *mut RawRuntime, spec: *const c_char, out: *mut *mut c_char) -> c_int;
    fn swb_gen_load(rt: *mut RawRuntime, id: *const c_char, spec: *const c_char, out: *mut u64) -> c_int;
    fn swb_gen_descriptor_json(rt: *mut RawRuntime, handle: u64, out: *mut *mut c_char) -> c_int;
    fn swb_gen_generate(rt: *mut RawRuntime, handle: u64, request: *const c_char, cb: EventCb, user: *mut c_void,
                        out: *mut *mut c_char) -> c_int;
    fn swb_gen_image_copy(rt: *mut RawRuntime, handle: u64, index: c_int, dst: *mut u8, capacity: usize) -> c_longlong;
    fn swb_handle_free(rt: *mut RawRuntime, handle: u64) -> c_int;
}

/// Error classes of the contracts (mirrors `enum swb_status`).
#[derive(Debug, Clone, PartialEq, Eq)]
pub enum Error {
    Invalid(String),
    Unsupported(String),
    Load(String),
    Canceled,
    Runtime(String),
    Python(String),
}

pub type Result<T> = std::result::Result<T, Error>;

fn last_error() -> String {
    unsafe { CStr::from_ptr(swb_rt_last_error()).to_string_lossy().into_owned() }
}

fn check(rc: c_int) -> Result<()> {
    match rc {
        0 => Ok(()),
        -1 => Err(Error::Invalid(last_error())),
        -2 => Err(Error::Unsupported(last_error())),
        -3 => Err(Error::Load(last_error())),
        -4 => Err(Error::Canceled),
        -6 => Err(Error::Python(last_error())),
        _ => Err(Error::Runtime(last_error())),
    }
}

unsafe fn take_json(p: *mut c_char) -> Result<Value> {
    if p.is_null() {
        return Ok(Value::Null);
    }
    let s = CStr::from_ptr(p).to_string_lossy().into_owned();
    swb_rt_free_string(p);
    serde_json::from_str(&s).map_err(|e| Error::Runtime(format!("malformed JSON from the runtime: {e}")))
}

fn cstring(s: &str) -> Result<CString> {
    CString::new(s).map_err(|_| Error::Invalid("string contains a NUL byte".into()))
}

/// The trampoline every callback goes through: `user` points at a `&mut dyn FnMut(&Value) -> bool` (true = go on).
unsafe extern "C" fn trampoline(js: *const c_char, user: *mut c_void) -> c_int {
    let f = &mut *(user as *mut &mut dyn FnMut(&Value) -> bool);
    let v: Value = serde_json::from_str(&CStr::from_ptr(js).to_string_lossy()).unwrap_or(Value::Null);
    if f(&v) { 0 } else { 1 }
}

/// A composed runtime bundle ("b200" or "cpu"). Dropping it closes the runtime.
pub struct Runtime {
    raw: *mut RawRuntime,
}

unsafe impl Send for Runtime {}

impl Runtime {
    /// `package_root`: directory containing the `inference_b200` Python package, or `None` if importable already.
    pub fn open(bundle: &str, package_root: Option<&str>) -> Result<Runtime> {
        let b = cstring(bundle)?;
        let root = package_root.map(cstring).transpose()?;
        let mut raw = ptr::null_mut();
        check(unsafe { swb_rt_open(b.as_ptr(), root.as_ref().map_or(ptr::null(), |r| r.as_ptr()), &mut raw) })?;
        Ok(Runtime { raw })
    }

    /// The catalog snapshot: platform, backend, generator ids, LLM ids, preparer backends, audio lane.
    pub fn catalog(&self) -> Result<Value> {
        let mut out = ptr::null_mut();
        check(unsafe { swb_rt_catalog_json(self.raw, &mut out) })?;
        unsafe { take_json(out) }
    }

    /// `provider_id = None` selects the provider by inspecting the model (the registry's `load_for_model`).
    pub fn load_text(&self, provider_id: Option<&str>, source: &str, quantize: Option<&str>) -> Result<TextLlm<'_>> {
        let pid = provider_id.map(cstring).transpose()?;
        let spec = cstring(&serde_json::json!({"source": source, "quantize": quantize}).to_string())?;
        let mut h = 0u64;
        check(unsafe {
            swb_text_load(self.raw, pid.as_ref().map_or(ptr::null(), |p| p.as_ptr()), spec.as_ptr(), &mut h)
        })?;
        Ok(TextLlm { rt: self, handle: h })
    }

    pub fn load_generator(&self, id: &str, weights_dir: &str, sequential_offload: bool) -> Result<Generator<'_>> {
        let gid = cstring(id)?;
        let policy = if sequential_offload { "sequential" } else { "resident" };
        let spec = cstring(&serde_json::json!({"weights": weights_dir, "offload_policy": policy}).to_string())?;
        let mut h = 0u64;
        check(unsafe { swb_gen_load(self.raw, gid.as_ptr(), spec.as_ptr(), &mut h) })?;
        Ok(Generator { rt: self, handle: h })
    }

    /// Snapshot preparation: `{"source", "out_dir", "quantize"}` -> report.
    pub fn prepare_snapshot(&self, source: &str, out_dir: &str, quantize: Option<&str>) -> Result<Value> {
        let spec = cstring(&serde_json::json!({"source": source, "out_dir": out_dir, "quantize": quantize}).to_string())?;
        let mut out = ptr::null_mut();
        check(unsafe { swb_prepare_snapshot(self.raw, spec.as_ptr(), &mut out) })?;
        unsafe { take_json(out) }
    }
}

impl Drop for Runtime {
    fn drop(&mut self) {
        unsafe { swb_rt_close(self.raw) }
    }
}

/// A loaded text LLM (the `TextLlm` contract).
pub struct TextLlm<'rt> {
    rt: &'rt Runtime,
    handle: u64,
}

impl TextLlm<'_> {
    pub fn descriptor(&self) -> Result<Value> {
        let mut out = ptr::null_mut();
        check(unsafe { swb_text_descriptor_json(self.rt.raw, self.handle, &mut out) })?;
        unsafe { take_json(out) }
    }

    /// `request`: `{"messages": [{"role", "content"}], "max_new_tokens", "temperature", "top_p", "seed", "stop",
    /// "json"}`. `on_event` sees `{"type": "token", ..}` / `{"type": "done", ..}`; returning false cancels.
    pub fn generate(&self, request: &Value, mut on_event: impl FnMut(&Value) -> bool) -> Result<Value> {
        let req = cstring(&request.to_string())?;
        let mut out = ptr::null_mut();
        let mut f: &mut dyn FnMut(&Value) -> bool = &mut on_event;
        let user = &mut f as *mut &mut dyn FnMut(&Value) -> bool as *mut c_void;
        check(unsafe { swb_text_generate(self.rt.raw, self.handle, req.as_ptr(), Some(trampoline), user, &mut out) })?;
        unsafe { take_json(out) }
    }

    pub fn complete(&self, request: &Value) -> Result<Value> {
        self.generate(request, |_| true)
    }
}

impl Drop for TextLlm<'_> {
    fn drop(&mut self) {
        unsafe { swb_handle_free(self.rt.raw, self.handle) };
    }
}

/// RGB8 image returned by a generator.
pub struct Image {
    pub width: u32,
    pub height: u32,
    pub pixels: Vec<u8>,
}

/// A loaded media generator (the `Generator` contract).
pub struct Generator<'rt> {
    rt: &'rt Runtime,
    handle: u64,
}

impl Generator<'_> {
    pub fn descriptor(&self) -> Result<Value> {
        let mut out = ptr::null_mut();
        check(unsafe { swb_gen_descriptor_json(self.rt.raw, self.handle, &mut out) })?;
        unsafe { take_json(out) }
    }

    /// `on_progress` sees `{"type": "loading" | "step" | "decoding", ..}`; returning false cancels.
    pub fn generate(&self, request: &Value, mut on_progress: impl FnMut(&Value) -> bool) -> Result<Vec<Image>> {
        let req = cstring(&request.to_string())?;
        let mut out = ptr::null_mut();
        let mut f: &mut dyn FnMut(&Value) -> bool = &mut on_progress;
        let user = &mut f as *mut &mut dyn FnMut(&Value) -> bool as *mut c_void;
        check(unsafe { swb_gen_generate(self.rt.raw, self.handle, req.as_ptr(), Some(trampoline), user, &mut out) })?;
        let meta = unsafe { take_json(out) }?;
        let mut images = Vec::new();
        for (i, m) in meta["images"].as_array().cloned().unwrap_or_default().iter().enumerate() {
            let n = m["bytes"].as_u64().unwrap_or(0) as usize;
            let mut pixels = vec![0u8; n];
            let got = unsafe { swb_gen_image_copy(self.rt.raw, self.handle, i as c_int, pixels.as_mut_ptr(), n) };
            if got < 0 {
                check(got as c_int)?;
            }
            images.push(Image { width: m["width"].as_u64().unwrap_or(0) as u32,
                                height: m["height"].as_u64().unwrap_or(0) as u32, pixels });
        }
        Ok(images)
    }
}

impl Drop for Generator<'_> {
    fn drop(&mut self) {
        unsafe { swb_handle_free(self.rt.raw, self.handle) };
    }
}
