// Links libvioletto_b200.so; VIOLETTO_B200_LIB_DIR names the directory that holds it (silicon-violetto_b200/ after
// `python silicon-violetto_b200/build.py`).
fn main() {
    println!("cargo:rerun-if-env-changed=VIOLETTO_B200_LIB_DIR");
    if let Ok(dir) = std::env::var("VIOLETTO_B200_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    }
    println!("cargo:rustc-link-lib=dylib=violetto_b200");
}
