// Points the linker at libautograph_b200.so.  AUTOGRAPH_B200_LIB_DIR names the directory that
// holds it (the `autograph_b200/` folder of this repository after `python -m autograph_b200.build`).
fn main() {
    if let Ok(dir) = std::env::var("AUTOGRAPH_B200_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    }
    println!("cargo:rustc-link-lib=dylib=autograph_b200");
    println!("cargo:rerun-if-env-changed=AUTOGRAPH_B200_LIB_DIR");
}
