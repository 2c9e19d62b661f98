//! Builds libmummu_cuda.so from the CUDA sources with nvcc for sm_100a and links it.
//! NOT COMPILED IN THIS REPOSITORY'S IMAGE (no Rust toolchain there); `python -m mummu_b200.build`
//! runs the same nvcc commands and is what the tests use.
use std::path::PathBuf;
use std::process::Command;

const SOURCES: &[&str] = &[
    "api.cu",
    "kernels_basic.cu",
    "decode_q4k.cu",
    "prefill_tc.cu",
    "trunk.cu",
    "ep.cu",
];

fn main() {
    let out = PathBuf::from(std::env::var("OUT_DIR").expect("OUT_DIR"));
    // the CUDA sources live beside the Python package in this repository
    let csrc = PathBuf::from(std::env::var("MUMMU_CUDA_CSRC").unwrap_or_else(|_| "../../mummu_b200/csrc".into()));
    let nvcc = std::env::var("NVCC").unwrap_or_else(|_| "nvcc".into());
    let mut objects = Vec::new();
    for src in SOURCES {
        let obj = out.join(src.replace(".cu", ".o"));
        let status = Command::new(&nvcc)
            .args([
                "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
                "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-c",
            ])
            .arg(csrc.join(src))
            .arg("-o")
            .arg(&obj)
            .status()
            .expect("nvcc not found: the CUDA toolkit (12.8 or later, for sm_100a) is required");
        assert!(status.success(), "nvcc failed on {src}");
        println!("cargo:rerun-if-changed={}", csrc.join(src).display());
        objects.push(obj);
    }
    let lib = out.join("libmummu_cuda.so");
    let status = Command::new(&nvcc)
        .arg("-shared")
        .arg("-o")
        .arg(&lib)
        .args(&objects)
        .args(["-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", "-lcudart", "-lcuda"])
        .status()
        .expect("nvcc link");
    assert!(status.success(), "nvcc link failed");
    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-lib=dylib=mummu_cuda");
}
