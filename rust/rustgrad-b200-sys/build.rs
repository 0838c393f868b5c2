//! Points the linker at `librg_b200.so`.  `RG_B200_LIB_DIR` names the directory that holds it (the
//! `rustgrad_b200/` folder of the repository after `python -m rustgrad_b200.build`).

fn main() {
    println!("cargo:rerun-if-env-changed=RG_B200_LIB_DIR");
    if let Ok(dir) = std::env::var("RG_B200_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    }
    println!("cargo:rustc-link-lib=dylib=rg_b200");
}
