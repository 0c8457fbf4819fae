// Points the linker at libcombskv.so.  COMBS_KV_LIB_DIR is the directory that holds it
// (combsengine_b200/ after `python -m combsengine_b200._build`).  Uncompiled here (no Rust toolchain).
fn main() {
    if let Ok(dir) = std::env::var("COMBS_KV_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
    }
    println!("cargo:rustc-link-lib=dylib=combskv");
    println!("cargo:rerun-if-env-changed=COMBS_KV_LIB_DIR");
}
