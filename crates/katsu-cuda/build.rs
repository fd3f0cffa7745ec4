// Builds libkatsu_cuda.so from the hand-written kernels with nvcc for sm_100a and links it.
//
// NOT COMPILED in the repository that carries the kernels (no Rust toolchain in its build image);
// the flags and the source set are the ones katsu_b200/build.py uses, which is what the tests run.
//
//   KATSU_CUDA_SRC   directory of the .cu / .cuh files   (default: ../../katsu_b200/csrc)
//   KATSU_CUDA_INC   directory of katsu_cuda.h           (default: ../../include)
//   KATSU_CUDA_LIB   a prebuilt libkatsu_cuda.so's directory: link it, compile nothing
//   NVCC             the compiler                        (default: nvcc on PATH, else /usr/local/cuda/bin/nvcc)
use std::env;
use std::path::{Path, PathBuf};
use std::process::Command;

const NVCC_FLAGS: &[&str] = &[
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
];

fn nvcc() -> String {
    if let Ok(path) = env::var("NVCC") {
        return path;
    }
    if Command::new("nvcc").arg("--version").output().is_ok() {
        return "nvcc".into();
    }
    "/usr/local/cuda/bin/nvcc".into()
}

fn run(cmd: &mut Command) {
    let status = cmd.status().unwrap_or_else(|e| panic!("cannot run {cmd:?}: {e}"));
    assert!(status.success(), "{cmd:?} failed");
}

fn main() {
    let manifest = PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap());
    println!("cargo:rerun-if-env-changed=KATSU_CUDA_LIB");
    if let Ok(dir) = env::var("KATSU_CUDA_LIB") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-lib=dylib=katsu_cuda");
        return;
    }
    let src = env::var("KATSU_CUDA_SRC").map(PathBuf::from).unwrap_or_else(|_| manifest.join("../../katsu_b200/csrc"));
    let inc = env::var("KATSU_CUDA_INC").map(PathBuf::from).unwrap_or_else(|_| manifest.join("../../include"));
    let out = PathBuf::from(env::var("OUT_DIR").unwrap());
    let nvcc = nvcc();

    // every .cu of the directory: the set is not spelled out here, so a new kernel file cannot be forgotten
    let mut sources: Vec<PathBuf> = std::fs::read_dir(&src)
        .unwrap_or_else(|e| panic!("cannot list {}: {e}", src.display()))
        .filter_map(|entry| entry.ok().map(|e| e.path()))
        .filter(|p| p.extension().map_or(false, |ext| ext == "cu"))
        .collect();
    sources.sort();
    assert!(!sources.is_empty(), "no .cu files in {}", src.display());
    for entry in std::fs::read_dir(&src).unwrap().flatten() {
        println!("cargo:rerun-if-changed={}", entry.path().display());
    }
    println!("cargo:rerun-if-changed={}", inc.join("katsu_cuda.h").display());

    let mut objects = Vec::new();
    for source in &sources {
        let object = out.join(Path::new(source.file_stem().unwrap()).with_extension("o"));
        run(Command::new(&nvcc)
            .args(NVCC_FLAGS)
            .arg("-I").arg(&inc)
            .arg("-I").arg(&src)
            .arg("-c").arg(source)
            .arg("-o").arg(&object));
        objects.push(object);
    }
    let library = out.join("libkatsu_cuda.so");
    run(Command::new(&nvcc).args(["-shared", "-cudart", "static", "-o"]).arg(&library).args(&objects).arg("-ldl"));
    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-lib=dylib=katsu_cuda");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", out.display());
}
