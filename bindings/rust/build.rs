// Links libswb200_capi.so. SWB200_LIB_DIR points at the directory holding it (inference_b200/_native in a source
// checkout); the directory is also baked into the rpath so binaries run without LD_LIBRARY_PATH.
fn main() {
    let dir = std::env::var("SWB200_LIB_DIR").unwrap_or_else(|_| "../../inference_b200/_native".to_string());
    println!("cargo:rustc-link-search=native={dir}");
    println!("cargo:rustc-link-lib=dylib=swb200_capi");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    println!("cargo:rerun-if-env-changed=SWB200_LIB_DIR");
}
