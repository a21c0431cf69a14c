// Link directive for librvllm_b200.so.  The directory comes from RVLLM_B200_LIB_DIR (the artifact
// directory `python -m rvllm_b200.build` writes, e.g. kernels_root/sm_100); nothing is compiled here.
fn main() {
    println!("cargo:rerun-if-env-changed=RVLLM_B200_LIB_DIR");
    if std::env::var_os("CARGO_FEATURE_DLOPEN_ONLY").is_some() {
        return;
    }
    if let Some(dir) = std::env::var_os("RVLLM_B200_LIB_DIR") {
        println!("cargo:rustc-link-search=native={}", std::path::Path::new(&dir).display());
    }
    println!("cargo:rustc-link-lib=dylib=rvllm_b200");
}
