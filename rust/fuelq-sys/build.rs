// Links libfuelq.so. FUELQ_LIB_DIR names the folder that holds it (the repository's fuel_b200/ after
// `python -c 'import __graft_entry__ as g; g.build()'`).
fn main() {
    if let Ok(dir) = std::env::var("FUELQ_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    }
    println!("cargo:rustc-link-lib=dylib=fuelq");
    println!("cargo:rerun-if-env-changed=FUELQ_LIB_DIR");
}
