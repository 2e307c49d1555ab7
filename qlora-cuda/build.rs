//! Links libqlora_cuda.so.  QLORA_CUDA_LIB_DIR names the directory that holds it (the in-tree build
//! leaves it in vkqlora/rs_b200/); the CUDA runtime it depends on is resolved by the dynamic loader.

use std::env;
use std::path::PathBuf;

fn main() {
    println!("cargo:rerun-if-env-changed=QLORA_CUDA_LIB_DIR");
    let dir = env::var("QLORA_CUDA_LIB_DIR")
        .map(PathBuf::from)
        .unwrap_or_else(|_| PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap()).join("../vkqlora/rs_b200"));
    println!("cargo:rustc-link-search=native={}", dir.display());
    println!("cargo:rustc-link-lib=dylib=qlora_cuda");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", dir.display());
}
