//! Links `libullis_cuda.so`.  `ULLIS_CUDA_LIB_DIR` names the directory that holds it (the
//! `ullis_b200/` directory of the CUDA backend's source tree after `python -m ullis_b200.build`);
//! the CUDA runtime is linked into the library statically and NCCL is resolved by the library
//! itself at run time, so nothing else has to be on the link line.
//! Uncompiled where this repository is developed: there is no rustc there.

fn main() {
    println!("cargo:rerun-if-env-changed=ULLIS_CUDA_LIB_DIR");
    if let Ok(dir) = std::env::var("ULLIS_CUDA_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        // so that `cargo run` finds the library without LD_LIBRARY_PATH
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    }
    println!("cargo:rustc-link-lib=dylib=ullis_cuda");
}
