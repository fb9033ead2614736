// Tells cargo where libirontimber_cuda.so lives.  IRONTIMBER_CUDA_LIB_DIR names the directory that holds the built
// library (python -m irontimber_b200.build writes it into irontimber_b200/); the default is that directory relative to
// this crate.  The library links the CUDA runtime statically; only the driver (libcuda.so.1) is resolved at run time.
use std::env;
use std::path::PathBuf;

fn main() {
    println!("cargo:rerun-if-env-changed=IRONTIMBER_CUDA_LIB_DIR");
    let dir = env::var("IRONTIMBER_CUDA_LIB_DIR").map(PathBuf::from).unwrap_or_else(|_| {
        PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap()).join("../../irontimber_b200")
    });
    println!("cargo:rustc-link-search=native={}", dir.display());
    println!("cargo:rustc-link-lib=dylib=irontimber_cuda");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", dir.display());
}
