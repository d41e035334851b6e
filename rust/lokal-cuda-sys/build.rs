// Links liblokal_cuda.so. LOKAL_CUDA_LIB_DIR names the directory that holds it (the `lokal_b200/` folder of the
// library's source tree after `python lokal_b200/_build.py`, or wherever it was installed).
fn main() {
    println!("cargo:rerun-if-env-changed=LOKAL_CUDA_LIB_DIR");
    if let Ok(dir) = std::env::var("LOKAL_CUDA_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    }
    println!("cargo:rustc-link-lib=dylib=lokal_cuda");
}
