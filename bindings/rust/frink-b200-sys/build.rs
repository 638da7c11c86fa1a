// Points the linker at libfrink_b200.so.  FRINK_B200_LIB_DIR names the directory that holds it
// (the `frink_b200/` package directory of a built checkout).
fn main() {
    println!("cargo:rerun-if-env-changed=FRINK_B200_LIB_DIR");
    if let Ok(dir) = std::env::var("FRINK_B200_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    }
    println!("cargo:rustc-link-lib=dylib=frink_b200");
}
