// Points the linker at libsagecuda.so: SAGE_CUDA_LIB_DIR, or ../../sage_b200 (the in-tree build).
fn main() {
    let dir = std::env::var("SAGE_CUDA_LIB_DIR").unwrap_or_else(|_| {
        let root = std::env::var("CARGO_MANIFEST_DIR").unwrap();
        format!("{root}/../../sage_b200")
    });
    println!("cargo:rustc-link-search=native={dir}");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    println!("cargo:rerun-if-env-changed=SAGE_CUDA_LIB_DIR");
}
