// Points the linker at libvfkv.so.  VFKV_LIB_DIR = the directory that holds it
// (vulkanforge_b200/ of the source tree after `python -m vulkanforge_b200.build`).
fn main() {
    if let Ok(dir) = std::env::var("VFKV_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
    }
    println!("cargo:rustc-link-lib=dylib=vfkv");
    println!("cargo:rerun-if-env-changed=VFKV_LIB_DIR");
}
