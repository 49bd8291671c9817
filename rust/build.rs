// Tells rustc where liblumen_b200.so lives: LUMEN_B200_LIB_DIR, or ../lumen_b200/lib (the in-tree build).
fn main() {
    let dir = std::env::var("LUMEN_B200_LIB_DIR").unwrap_or_else(|_| {
        let here = std::env::var("CARGO_MANIFEST_DIR").unwrap();
        format!("{}/../lumen_b200/lib", here)
    });
    println!("cargo:rustc-link-search=native={}", dir);
    println!("cargo:rustc-link-lib=dylib=lumen_b200");
    println!("cargo:rerun-if-env-changed=LUMEN_B200_LIB_DIR");
}
