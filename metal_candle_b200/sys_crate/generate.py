"""Writes the Rust `-sys` crate source for libmetal_candle_b200.so from include/mcb200.h.

    python metal_candle_b200/sys_crate/generate.py [--check]

The crate (Cargo.toml, build.rs, src/lib.rs next to this file) is what a maintainer of the reference adds to bind
the library: one `extern "C"` declaration per exported entry point, the `#[repr(C)]` AdamW descriptor and the
status / option constants.  It is generated so that it cannot drift from the header; tests/test_abi.py runs
`--check`.  There is no Rust toolchain where this library is built, so the crate is source only: it has never
been compiled.
"""
from __future__ import annotations

import re
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
HEADER = HERE.parent.parent / "include" / "mcb200.h"
OUT = HERE / "src" / "lib.rs"

TYPES = {
    "void": None, "int": "c_int", "float": "f32", "double": "f64", "int64_t": "i64", "int32_t": "i32", "uint64_t": "u64",
    "size_t": "usize", "char": "c_char", "mcb_adamw_tensor": "mcb_adamw_tensor", "mcb_comm": "mcb_comm",
    "mcb_lora_segment": "mcb_lora_segment", "mcb_qwen": "mcb_qwen", "mcb_qwen_config": "mcb_qwen_config",
    "mcb_qwen_weights": "mcb_qwen_weights", "mcb_qwen_adapter_entry": "mcb_qwen_adapter_entry",
}


def rust_type(c: str) -> str:
    c = c.strip()
    const = c.startswith("const ")
    if const:
        c = c[len("const "):].strip()
    stars = c.count("*")
    base = c.replace("*", "").strip()
    if base not in TYPES:
        raise SystemExit(f"generate.py: no Rust mapping for C type '{c}'")
    t = TYPES[base] or "c_void"
    if stars == 0:
        if base == "void":
            raise SystemExit("generate.py: bare void parameter")
        return t
    out = t
    for level in range(stars):
        innermost = level == 0
        out = ("*const " if (const and innermost) else "*mut ") + out
    return out


def parse(header: str):
    text = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    consts = []
    for m in re.finditer(r"^#define\s+(MCB_[A-Z0-9_]+)\s+(\(?-?\d+\)?)\s*$", text, flags=re.M):
        name, val = m.group(1), m.group(2).strip("()")
        if name.endswith("_"):
            continue
        consts.append((name, int(val)))
    funcs = []
    for m in re.finditer(r"^([A-Za-z_][A-Za-z0-9_ \*]*?)\s*\b(mcb_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", text, flags=re.M | re.S):
        ret, name, args = m.group(1).strip(), m.group(2), " ".join(m.group(3).split())
        params = []
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                pm = re.match(r"^(.*?)([A-Za-z_][A-Za-z0-9_]*)$", a)
                params.append((pm.group(2), rust_type(pm.group(1))))
        rret = None if ret == "void" else rust_type(ret)
        funcs.append((name, params, rret))
    return consts, funcs


RESERVED = {"type", "ref", "in", "loop", "move", "fn", "box", "where", "impl", "match", "mod", "use", "self"}


def render(consts, funcs) -> str:
    lines = [
        "//! Raw bindings to libmetal_candle_b200.so, the B200 (sm_100a) kernels behind metal-candle's custom-op hot path.",
        "//!",
        "//! GENERATED from include/mcb200.h by metal_candle_b200/sys_crate/generate.py - do not edit.  The header",
        "//! documents every entry point (which reference interface it replaces, argument layouts, error codes).",
        "//! All pointers are CUDA device pointers owned by the caller unless the header says otherwise; every call",
        "//! returns a status (`MCB_OK` = 0) and enqueues its work on the given `cudaStream_t` (passed as `*mut c_void`).",
        "//!",
        "//! This crate has never been compiled: the machines the library is built on carry no Rust toolchain.",
        "#![allow(non_camel_case_types, non_snake_case)]",
        "",
        "use core::ffi::{c_char, c_int, c_void};",
        "",
    ]
    for name, val in consts:
        lines.append(f"pub const {name}: c_int = {val};")
    lines += [
        "",
        "/// `MCB_COMM_NO_STREAM`: wait on the communicator's own state only.",
        "pub const MCB_COMM_NO_STREAM: *mut c_void = usize::MAX as *mut c_void;",
        "",
        "/// One tensor of an `mcb_adamw_multi` call (a HOST array of these is passed).",
        "#[repr(C)]",
        "#[derive(Debug, Clone, Copy)]",
        "pub struct mcb_adamw_tensor {",
        "    pub p: *mut f32,",
        "    pub g: *const f32,",
        "    pub m: *mut f32,",
        "    pub v: *mut f32,",
        "    pub n: i64,",
        "    pub t: i32,",
        "    pub pad_: i32,",
        "}",
        "",
        "/// One projection of a fused linear (`mcb_lora_linear_fused_*`; a HOST array of these is passed).",
        "#[repr(C)]",
        "#[derive(Debug, Clone, Copy)]",
        "pub struct mcb_lora_segment {",
        "    pub A: *const f32,",
        "    pub B: *const f32,",
        "    pub dA: *mut f32,",
        "    pub dB: *mut f32,",
        "    pub n_offset: i64,",
        "    pub n: i64,",
        "}",
        "",
        "/// The model's shape (`mcb_qwen_*`).",
        "#[repr(C)]",
        "#[derive(Debug, Clone, Copy)]",
        "pub struct mcb_qwen_config {",
        "    pub vocab_size: i64,",
        "    pub hidden_size: i64,",
        "    pub intermediate_size: i64,",
        "    pub num_layers: i64,",
        "    pub num_heads: i64,",
        "    pub num_kv_heads: i64,",
        "    pub rms_norm_eps: f32,",
        "    pub rope_theta: f32,",
        "}",
        "",
        "/// One decoder layer's bf16 device tensors, weights in [out, in] layout, by module q k v o gate up down.",
        "#[repr(C)]",
        "#[derive(Debug, Clone, Copy)]",
        "pub struct mcb_qwen_layer {",
        "    pub input_layernorm: *const c_void,",
        "    pub post_attention_layernorm: *const c_void,",
        "    pub weight: [*const c_void; 7],",
        "    pub bias: [*const c_void; 3],",
        "}",
        "",
        "#[repr(C)]",
        "#[derive(Debug, Clone, Copy)]",
        "pub struct mcb_qwen_weights {",
        "    pub embed_tokens: *const c_void,",
        "    pub final_norm: *const c_void,",
        "    pub lm_head: *const c_void,",
        "    pub layers: *const mcb_qwen_layer,",
        "}",
        "",
        "#[repr(C)]",
        "#[derive(Debug, Clone, Copy)]",
        "pub struct mcb_qwen_adapter_entry {",
        "    pub layer: i32,",
        "    pub module: i32,",
        "    pub A: *const f32,",
        "    pub B: *const f32,",
        "    pub dA: *mut f32,",
        "    pub dB: *mut f32,",
        "}",
        "",
        "/// Opaque training-step engine (`mcb_qwen_*`).",
        "#[repr(C)]",
        "pub struct mcb_qwen {",
        "    _private: [u8; 0],",
        "}",
        "",
        "/// Opaque communicator handle (`mcb_comm_*`).",
        "#[repr(C)]",
        "pub struct mcb_comm {",
        "    _private: [u8; 0],",
        "}",
        "",
        '#[link(name = "metal_candle_b200")]',
        'extern "C" {',
    ]
    for name, params, ret in funcs:
        ps = ", ".join(f"{(p + '_') if p in RESERVED else p}: {t}" for p, t in params)
        lines.append(f"    pub fn {name}({ps})" + (f" -> {ret};" if ret else ";"))
    lines += ["}", ""]
    return "\n".join(lines)


def main() -> int:
    consts, funcs = parse(HEADER.read_text())
    src = render(consts, funcs)
    if "--check" in sys.argv:
        if not OUT.exists() or OUT.read_text() != src:
            print(f"{OUT} is out of date: run python {Path(__file__).name}", file=sys.stderr)
            return 1
        return 0
    OUT.parent.mkdir(parents=True, exist_ok=True)
    OUT.write_text(src)
    print(f"wrote {OUT} ({len(funcs)} functions, {len(consts)} constants)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
