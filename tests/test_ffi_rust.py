"""CPU: the Rust crate's ffi.rs (rust/nabla-optim-b200/src/ffi.rs) against include/nabla_optim_b200.h,
declaration by declaration.  No Rust toolchain is needed: the header is parsed independently of the
generator's own parser, ffi.rs is parsed as text, and the two must agree on every function name, argument
count, argument names, pointer depth and constness, on every struct's fields and on every enumerator."""
import importlib.util
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "nabla_optim_b200.h")
CRATE = os.path.join(ROOT, "rust", "nabla-optim-b200")
FFI = os.path.join(CRATE, "src", "ffi.rs")


def header_functions():
    """{name: [(arg name, pointer depth, base C type, pointee-of-outermost-pointer is const)]}"""
    src = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    src = "\n".join(l for l in src.splitlines() if not l.strip().startswith("#"))
    out = {}
    for m in re.finditer(r"NBO_API\s+([^;]*?)\b(nbo_\w+)\s*\(([^;]*?)\)\s*;", src, flags=re.S):
        args = " ".join(m.group(3).split())
        params = []
        if args != "void":
            for a in args.split(","):
                a = a.strip()
                arr = re.search(r"\[\s*\d+\s*\]$", a)
                if arr:
                    a = a[:arr.start()].rstrip()
                name = re.search(r"(\w+)$", a).group(1)
                ctype = a[:-len(name)].strip()
                depth = ctype.count("*") + (1 if arr else 0)
                base = [t for t in re.sub(r"[*]", " ", ctype).split() if t != "const"][0]
                params.append((name, depth, base))
        out[m.group(2)] = params
    return out


def rust_functions():
    text = open(FFI).read()
    block = text[text.index('extern "C" {'):]
    out = {}
    for m in re.finditer(r"pub fn (\w+)\((.*?)\) -> ([^;]+);", block):
        params = []
        if m.group(2).strip():
            for a in m.group(2).split(", "):
                name, ty = a.split(": ", 1)
                depth = ty.count("*const ") + ty.count("*mut ")
                base = ty.replace("*const ", "").replace("*mut ", "").strip()
                params.append((name, depth, base))
        out[m.group(1)] = params
    return out


C_TO_RUST = {"int32_t": "i32", "uint32_t": "u32", "uint64_t": "u64", "double": "f64", "float": "f32", "uint8_t": "u8",
             "char": "c_char", "void": "c_void", "nbo_optimizer": "NboOptimizer", "nbo_symm": "NboSymm", "nbo_group_config": "NboGroupConfig",
             "nbo_scaler_state": "NboScalerState", "nbo_lr_schedule": "NboLrSchedule", "nbo_step_result": "NboStepResult"}


def test_every_header_declaration_has_its_rust_line():
    hdr, rs = header_functions(), rust_functions()
    assert len(hdr) >= 49
    assert sorted(hdr) == sorted(rs), (sorted(set(hdr) ^ set(rs)))
    for name, params in hdr.items():
        got = rs[name]
        assert len(got) == len(params), f"{name}: {len(got)} Rust arguments for {len(params)} in the header"
        for (cn, cdepth, cbase), (rn, rdepth, rbase) in zip(params, got):
            assert (cn, cdepth, C_TO_RUST[cbase]) == (rn, rdepth, rbase), (name, cn, rn)


def test_ffi_rs_is_what_the_generator_writes():
    spec = importlib.util.spec_from_file_location("gen_ffi", os.path.join(CRATE, "gen_ffi.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    assert gen.generate(open(HEADER).read()) == open(FFI).read(), "run rust/nabla-optim-b200/gen_ffi.py"


def test_constness_and_structs():
    rs = open(FFI).read()
    # spot checks of pointer constness, which the name/depth comparison above does not see
    assert "pub fn nbo_step(h: *mut NboOptimizer, n: u64, params: *const *mut c_void, grads: *const *const c_void) -> i32;" in rs
    assert "pub fn nbo_last_error(h: *const NboOptimizer) -> *const c_char;" in rs
    assert "pub fn nbo_zero1_unique_id(id_out: *mut u8) -> i32;" in rs
    assert "unique_id: *const u8) -> i32;" in rs
    src = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    for body, cname in re.findall(r"typedef\s+struct\s*\{(.*?)\}\s*(\w+)\s*;", src, flags=re.S):
        fields = [re.search(r"(\w+)$", " ".join(f.split())).group(1) for f in body.split(";") if f.strip()]
        rbody = re.search(r"pub struct %s \{(.*?)\}" % C_TO_RUST[cname], rs, flags=re.S).group(1)
        assert re.findall(r"pub (\w+):", rbody) == fields, cname
    for k, v in re.findall(r"\b(NBO_\w+)\s*=\s*(\d+)", src):
        assert f"pub const {k}: i32 = {v};" in rs


def test_lib_rs_uses_only_declared_functions_and_covers_the_traits():
    lib = open(os.path.join(CRATE, "src", "lib.rs")).read()
    declared = set(rust_functions())
    used = set(re.findall(r"\b(nbo_\w+)\(", lib))
    assert used <= declared, used - declared
    for ty in ("B200Sgd", "B200Adam", "B200AdamW", "B200GroupOptimizer", "B200MixedAdamW"):
        assert re.search(r"pub struct %s\b" % ty, lib) or f"single_group_optimizer!({ty}," in lib, ty
    assert lib.count("impl Optimizer<f32, Cuda> for") == 2       # the macro (three types) and the group optimizer
    assert lib.count("impl OptimState<f32, Cuda> for") == 3      # the macro, the group optimizer, the mixed optimizer
    assert lib.count("pub fn zero_grad") == 3
