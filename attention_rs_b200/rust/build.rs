// Build script of the `kernels` crate when it links the sm_100a library instead of
// compiling the reference's .cu files (replaces src/kernels/build.rs:1-32 of the reference).
//
// NOT COMPILED in the environment this repository was developed in (no cargo / rustc there);
// it is the recipe a maintainer of the reference would drop in.
//
// It compiles every .cu under PA_B200_CSRC with nvcc for sm_100a ONLY (no other architecture,
// no Metal, no CPU fallback) into libpagedattention_b200.a and links cudart.
use std::env;
use std::path::PathBuf;
use std::process::Command;

fn main() {
    println!("cargo:rerun-if-changed=build.rs");
    let csrc = PathBuf::from(env::var("PA_B200_CSRC").unwrap_or_else(|_| "../csrc".to_string()));
    let out = PathBuf::from(env::var("OUT_DIR").expect("OUT_DIR"));
    let mut objects = Vec::new();
    for entry in std::fs::read_dir(&csrc).expect("csrc directory") {
        let path = entry.expect("dir entry").path();
        if path.extension().map(|e| e == "cu").unwrap_or(false) {
            println!("cargo:rerun-if-changed={}", path.display());
            let obj = out.join(path.file_stem().unwrap()).with_extension("o");
            let status = Command::new("nvcc")
                .args(["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo"])
                .args(["-Xcompiler", "-fPIC", "-c"])
                .arg(&path)
                .arg("-o")
                .arg(&obj)
                .status()
                .expect("nvcc not found");
            assert!(status.success(), "nvcc failed on {}", path.display());
            objects.push(obj);
        }
    }
    let lib = out.join("libpagedattention_b200.a");
    let status = Command::new("ar").arg("crs").arg(&lib).args(&objects).status().expect("ar");
    assert!(status.success());
    println!("cargo:rustc-link-search={}", out.display());
    println!("cargo:rustc-link-lib=static=pagedattention_b200");
    println!("cargo:rustc-link-lib=dylib=cudart");
    println!("cargo:rustc-link-lib=dylib=stdc++");
}
