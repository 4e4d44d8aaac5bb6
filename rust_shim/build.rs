// Links liblumi_b200.so (built by `python -m lumi_b200.build` with nvcc for sm_100a only).
fn main() {
    let dir = std::env::var("LUMI_B200_LIB_DIR").expect("set LUMI_B200_LIB_DIR to <repo>/lumi_b200/lib");
    println!("cargo:rustc-link-search=native={dir}");
    println!("cargo:rustc-link-lib=dylib=lumi_b200");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    println!("cargo:rerun-if-env-changed=LUMI_B200_LIB_DIR");
}
