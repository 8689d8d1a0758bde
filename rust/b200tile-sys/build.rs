// Points the linker at libb200tile.so: B200TILE_LIB_DIR, or cutile_rs_b200/ of this repository.
use std::path::PathBuf;

fn main() {
    let dir = std::env::var("B200TILE_LIB_DIR").map(PathBuf::from).unwrap_or_else(|_| {
        PathBuf::from(std::env::var("CARGO_MANIFEST_DIR").unwrap()).join("../../cutile_rs_b200")
    });
    println!("cargo:rustc-link-search=native={}", dir.display());
    println!("cargo:rustc-link-lib=dylib=b200tile");
    println!("cargo:rerun-if-env-changed=B200TILE_LIB_DIR");
    println!("cargo:rerun-if-changed=../../include/b200tile.h");
}
