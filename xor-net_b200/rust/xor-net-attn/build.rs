// Compiles the CUDA library for sm_100a with nvcc and links it statically.
// XN_ATTN_ROOT points at the repository root (contains include/ and xor-net_b200/csrc/).
use std::{env, path::PathBuf, process::Command};

fn main() {
    let root = PathBuf::from(env::var("XN_ATTN_ROOT").unwrap_or_else(|_| "../../..".into()));
    let out = PathBuf::from(env::var("OUT_DIR").unwrap());
    let obj = out.join("xn_attn.o");
    let status = Command::new("nvcc")
        .args(["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
               "-Xcompiler", "-fPIC", "-c"])
        .arg("-I").arg(root.join("include"))
        .arg(root.join("xor-net_b200/csrc/xn_attn.cu"))
        .arg("-o").arg(&obj)
        .status()
        .expect("nvcc not found");
    assert!(status.success(), "nvcc failed");
    let lib = out.join("libxn_attn.a");
    assert!(Command::new("ar").arg("crs").arg(&lib).arg(&obj).status().unwrap().success());
    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-lib=static=xn_attn");
    let cuda = env::var("CUDA_HOME").unwrap_or_else(|_| "/usr/local/cuda".into());
    println!("cargo:rustc-link-search=native={}/lib64", cuda);
    println!("cargo:rustc-link-lib=cudart");
    println!("cargo:rustc-link-lib=stdc++");
    println!("cargo:rerun-if-changed={}", root.join("xor-net_b200/csrc").display());
}
