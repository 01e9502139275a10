// Builds libtile_sm100.so with nvcc for sm_100a and links it.  The same command lines as
// tile-rs_b200/build.py; TILE_SM100_ROOT points at a checkout of this repository
// (default: two directories up from this crate).
use std::{env, path::PathBuf, process::Command};

fn main() {
    let root = env::var("TILE_SM100_ROOT").map(PathBuf::from).unwrap_or_else(|_| {
        PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap()).join("../..")
    });
    let csrc = root.join("tile-rs_b200/csrc");
    let include = root.join("include");
    let out = PathBuf::from(env::var("OUT_DIR").unwrap());
    let nvcc = env::var("NVCC").unwrap_or_else(|_| "nvcc".into());
    let common = [
        "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-fopenmp",
    ];
    let mut objects = Vec::new();
    for src in ["runtime.cu", "capi_ops.cu", "multi.cu", "inputs.cpp", "emit.cpp"] {
        let obj = out.join(format!("{src}.o"));
        let mut cmd = Command::new(&nvcc);
        cmd.args(common).arg(format!("-I{}", include.display()));
        if src.ends_with(".cpp") {
            cmd.args(["-x", "cu"]);
        }
        cmd.arg("-c").arg(csrc.join(src)).arg("-o").arg(&obj);
        assert!(cmd.status().expect("nvcc not found").success(), "nvcc failed on {src}");
        objects.push(obj);
        println!("cargo:rerun-if-changed={}", csrc.join(src).display());
    }
    for header in std::fs::read_dir(&csrc).unwrap().flatten() {
        println!("cargo:rerun-if-changed={}", header.path().display());
    }
    println!("cargo:rerun-if-changed={}", include.join("tile_sm100.h").display());
    let lib = out.join("libtile_sm100.so");
    let mut link = Command::new(&nvcc);
    link.arg("-shared").arg("-o").arg(&lib).args(&objects)
        .args(["-cudart", "static", "-Xcompiler", "-fopenmp", "-ldl"]);
    assert!(link.status().unwrap().success(), "linking libtile_sm100.so failed");
    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-lib=dylib=tile_sm100");
    // the emitted kernel modules #include the kernel headers: tell dependants where they are
    println!("cargo:csrc={}", csrc.display());
    println!("cargo:include={}", include.display());
}
