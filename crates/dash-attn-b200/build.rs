//! Compiles the hand-written CUDA sources for sm_100a with nvcc and links them into the crate.
//!
//! `DASH_ATTN_CSRC` names the directory that holds them (`dashmag_b200/csrc` of the B200 repository,
//! with `include/dash_attn.h` two levels up, as the sources include it); `NVCC` overrides the
//! compiler.  No CubeCL, no Triton, no other backend: this is the only device code of the crate.
use std::{env, path::PathBuf, process::Command};

const SOURCES: &[&str] = &[
    "api.cu",
    "generic_train.cu",
    "decode.cu",
    "rope.cu",
    "sample.cu",
    "sm100.cu",
    "fwd_sm100.cu",
    "fwd2_sm100.cu",
    "bwd_sm100.cu",
    "bwd256_sm100.cu",
];

fn main() {
    let out = PathBuf::from(env::var("OUT_DIR").expect("OUT_DIR"));
    let csrc = PathBuf::from(env::var("DASH_ATTN_CSRC").unwrap_or_else(|_| "csrc".into()));
    let nvcc = env::var("NVCC").unwrap_or_else(|_| "nvcc".into());
    println!("cargo:rerun-if-env-changed=DASH_ATTN_CSRC");
    println!("cargo:rerun-if-env-changed=NVCC");
    let mut objects = Vec::new();
    for source in SOURCES {
        let path = csrc.join(source);
        println!("cargo:rerun-if-changed={}", path.display());
        let object = out.join(source).with_extension("o");
        let status = Command::new(&nvcc)
            .args(["-gencode", "arch=compute_100a,code=sm_100a"])
            .args(["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr"])
            .args(["-Xcompiler", "-fPIC", "-c"])
            .arg(&path)
            .arg("-o")
            .arg(&object)
            .status()
            .unwrap_or_else(|e| panic!("{nvcc}: {e}"));
        assert!(status.success(), "nvcc failed on {}", path.display());
        objects.push(object);
    }
    for header in ["common.cuh", "bwd_common.cuh", "sm100_ptx.cuh", "sm100_kernels.h", "sm100.h", "launch.h", "rope.h", "sample.h"] {
        println!("cargo:rerun-if-changed={}", csrc.join(header).display());
    }
    let archive = out.join("libdash_attn_b200.a");
    let status = Command::new("ar").arg("crs").arg(&archive).args(&objects).status().expect("ar");
    assert!(status.success(), "ar failed");
    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-lib=static=dash_attn_b200");
    // The CUDA runtime the objects were compiled against, and the C++ runtime of the host code.
    if let Ok(cuda) = env::var("CUDA_HOME").or_else(|_| env::var("CUDA_PATH")) {
        println!("cargo:rustc-link-search=native={cuda}/lib64");
    }
    println!("cargo:rustc-link-lib=dylib=cudart");
    println!("cargo:rustc-link-lib=dylib=stdc++");
}
