// Links the prebuilt C-ABI library. ARGUS_B200_LIB_DIR points at the directory holding libargus_b200.so
// (built by `python -m argus_engine_b200.build`).
fn main() {
    if let Ok(dir) = std::env::var("ARGUS_B200_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
    }
    println!("cargo:rustc-link-lib=dylib=argus_b200");
    println!("cargo:rerun-if-env-changed=ARGUS_B200_LIB_DIR");
}
