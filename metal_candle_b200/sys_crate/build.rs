// Tells rustc where libmetal_candle_b200.so lives.  MCB200_LIB_DIR names the directory that holds the shared
// library built by `python -m metal_candle_b200.build` (nvcc, sm_100a); by default the package directory two levels
// above this crate.
use std::env;
use std::path::PathBuf;

fn main() {
    let dir = env::var("MCB200_LIB_DIR").map(PathBuf::from).unwrap_or_else(|_| {
        PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap()).join("..")
    });
    println!("cargo:rustc-link-search=native={}", dir.display());
    println!("cargo:rustc-link-lib=dylib=metal_candle_b200");
    println!("cargo:rerun-if-env-changed=MCB200_LIB_DIR");
}
