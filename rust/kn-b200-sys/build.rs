// Links libkn_b200.so.  KN_B200_LIB_DIR names the directory that holds it (the `kyanite_b200/` folder of the
// repository after `python -m kyanite_b200.build`).  The library links the CUDA runtime statically and
// resolves the driver and NCCL at run time, so nothing else is needed at link time.
use std::env;

fn main() {
    println!("cargo:rerun-if-env-changed=KN_B200_LIB_DIR");
    let dir = env::var("KN_B200_LIB_DIR").expect("set KN_B200_LIB_DIR to the directory that contains libkn_b200.so");
    println!("cargo:rustc-link-search=native={}", dir);
    println!("cargo:rustc-link-lib=dylib=kn_b200");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", dir);
}
