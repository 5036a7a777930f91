"""The Rust side of the boundary is source only (no rustc where this is developed), so what can be
checked is checked by reading: the `ullis-cuda-sys` declarations against include/ullis_cuda.h - every
name, the number of arguments, and the kind and width of each argument and return value - and every
`sys::` item `src/cuda.rs` uses against those declarations."""
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SYS = os.path.join(ROOT, "rust", "ullis-cuda-sys")

# C type -> (pointer depth, pointee constness, scalar kind) and the same for the Rust spelling
C_SCALAR = {"int32_t": "i32", "uint32_t": "u32", "uint64_t": "u64", "uint16_t": "u16", "uint8_t": "u8", "size_t": "usize",
            "float": "f32", "double": "f64", "char": "c_char", "void": "c_void"}


def c_declarations():
    text = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "ullis_cuda.h")).read(), flags=re.S)
    out = {}
    for m in re.finditer(r"ULLIS_CUDA_API\s+([\w\s\*]+?)\b(ullis_cuda_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
        ret, name, args = m.group(1).strip(), m.group(2), " ".join(m.group(3).split())
        params = []
        for a in ([] if args in ("", "void") else args.split(",")):
            a = a.strip()
            am = re.match(r"(.+?)\b(\w+)\s*(\[\d*\])?$", a)
            params.append(c_kind(am.group(1), am.group(3) is not None))
        out[name] = (None if ret == "void" else c_kind(ret, False), params)
    return out


def c_kind(ctype, array):
    ctype = ctype.strip()
    const = ctype.startswith("const ")
    base = ctype.replace("const ", "").replace("*", "").strip()
    depth = ctype.count("*") + (1 if array else 0)
    return (depth, const and depth > 0, C_SCALAR.get(base, base))


def rust_kind(rtype):
    rtype = rtype.strip()
    depth, const = 0, False
    first = True
    while rtype.startswith("*"):
        is_const = rtype.startswith("*const ")
        rtype = rtype[len("*const "):] if is_const else rtype[len("*mut "):]
        depth += 1
        const = is_const      # constness of the innermost pointee is spelled last
        first = False
    return (depth, const, rtype.strip())


def rust_declarations():
    text = open(os.path.join(SYS, "src", "lib.rs")).read()
    block = text[text.index('unsafe extern "C" {'):]
    out = {}
    for m in re.finditer(r"pub fn (ullis_cuda_\w+)\s*\((.*?)\)\s*(?:->\s*([^;]+))?;", block, flags=re.S):
        name, args, ret = m.group(1), " ".join(m.group(2).split()), m.group(3)
        params = [rust_kind(a.split(":", 1)[1]) for a in args.split(",") if ":" in a]
        out[name] = (rust_kind(ret) if ret else None, params)
    return out


def test_sys_crate_is_generated_from_the_header():
    assert subprocess.run([sys.executable, os.path.join(SYS, "gen_bindings.py"), "--check"]).returncode == 0


def test_every_header_declaration_has_a_rust_twin_of_the_same_shape():
    c, r = c_declarations(), rust_declarations()
    assert len(c) >= 60 and set(c) == set(r)
    for name, (ret, params) in c.items():
        r_ret, r_params = r[name]
        assert (ret is None) == (r_ret is None), name
        if ret is not None:
            assert ret[0] == r_ret[0] and ret[2] == r_ret[2], (name, ret, r_ret)
        assert len(params) == len(r_params), name
        for i, (cp, rp) in enumerate(zip(params, r_params)):
            assert cp == rp, (name, i, cp, rp)     # pointer depth, const-ness of the pointee, scalar width


def test_cuda_rs_only_calls_what_the_header_declares_with_the_right_argument_count():
    text = open(os.path.join(ROOT, "rust", "src", "cuda.rs")).read()
    text = re.sub(r"//.*", "", text)
    decl = rust_declarations()
    sys_text = open(os.path.join(SYS, "src", "lib.rs")).read()
    used = set()
    for m in re.finditer(r"sys::(ullis_cuda_\w+)\s*\(", text):
        name = m.group(1)
        assert name in decl, name
        used.add(name)
        # the argument list up to the matching parenthesis
        depth, i = 1, m.end()
        start = i
        while depth:
            depth += {"(": 1, ")": -1}.get(text[i], 0)
            i += 1
        args = text[start:i - 1]
        # top-level commas
        n, d = (1 if args.strip() else 0), 0
        for ch in args.rstrip().rstrip(","):
            d += {"(": 1, "[": 1, ")": -1, "]": -1}.get(ch, 0)
            n += ch == "," and d == 0
        assert n == len(decl[name][1]), (name, n, len(decl[name][1]))
    for m in re.finditer(r"sys::(ULLIS_CUDA_\w+|ullis_cuda_\w+)", text):     # constants and struct names exist too
        assert re.search(r"\b" + m.group(1) + r"\b", sys_text), m.group(1)
    # the wrapper reaches the whole forward path, the model, generation, training and the group calls
    for needed in ("ullis_cuda_model_forward_ce", "ullis_cuda_layer_norm", "ullis_cuda_binary_linear",
                   "ullis_cuda_rosa_qkv_1bit_fwd", "ullis_cuda_rosa_block_forward", "ullis_cuda_cmix_block_forward",
                   "ullis_cuda_streamed_ce", "ullis_cuda_generate_step", "ullis_cuda_model_train_step",
                   "ullis_cuda_model_read_loss_global", "ullis_cuda_dp_init"):
        assert needed in used, needed


def test_metal_runtime_method_names_are_mirrored():
    """The methods of the reference's MetalRuntime that lie on the forward / CE / optimiser path, by name."""
    text = open(os.path.join(ROOT, "rust", "src", "cuda.rs")).read()
    for method in ("synchronize", "residual_add", "time_shift_delta", "sign_pack_bits", "rosa_qkv_1bit_fwd",
                   "rosa_qkv_1bit_bwd_e", "rosa_block_forward", "cmix_relu2", "cmix_relu2_backward", "layer_norm",
                   "layer_norm_backward", "binary_linear", "cmix_block_forward", "fp16_linear",
                   "streamed_cross_entropy_fp16", "apply_latent_sgd", "clipped_sgd_fp16", "binaryconnect_sgd_fp16"):
        assert re.search(r"pub fn " + method + r"\b", text), method
