// Links the ahead-of-time built CUDA library.  NABLA_OPTIM_B200_LIB_DIR names the directory that holds
// libnabla_optim_b200.so (built by `make -C nabla_b200/csrc`); by default the in-tree location is used.
use std::env;
use std::path::PathBuf;

fn main() {
    let dir = env::var("NABLA_OPTIM_B200_LIB_DIR").map(PathBuf::from).unwrap_or_else(|_| {
        PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap()).join("../../nabla_b200")
    });
    println!("cargo:rustc-link-search=native={}", dir.display());
    println!("cargo:rustc-link-lib=dylib=nabla_optim_b200");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", dir.display());
    println!("cargo:rerun-if-env-changed=NABLA_OPTIM_B200_LIB_DIR");
    println!("cargo:rerun-if-changed=../../include/nabla_optim_b200.h");
}
