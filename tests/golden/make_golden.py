"""Generate the golden vectors under tests/golden from the reference's own CPU emulation.

Run in the build container only (it needs the reference checkout):

    python tests/golden/make_golden.py --reference <path of the reference checkout>

It loads ``transformer_engine/pytorch/custom_recipes/quantization_nvfp4.py`` (and its two
small helper modules) straight from the reference tree, with stub parents injected into
``sys.modules`` because the compiled ``transformer_engine`` package is not installable here.
A second fixture, ``rmsnorm_bwd_reference_golden.npz``, comes from the reference's PyTorch formula for the
RMSNorm backward of the FFN block (one function executed out of ``fused_te_linear.py``); a third,
``scale_swizzle_reference_golden.npz``, from the torch helper of the reference's MXFP4 tests that lays scale
bytes out in 512-byte tiles; a fourth, ``mxfp4_reference_golden.npz``, from the MXFP4 emulation
(``custom_recipes/quantization_mxfp4.py``); a fifth, ``tk_gemm_quantize_reference_golden.npz``, from the torch
reference of the GEMM module's own tile quantiser (its ``test_quantize.py``); a sixth,
``rht_and_norm_reference_golden.npz``, from the emulation's Hadamard transform and the PyTorch formula of the
forward RMSNorm.
Nothing from the reference is copied into this repository: only seeded inputs (as bf16 bit
patterns) and the bytes the reference produced for them are stored.
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(root: str):
    base = os.path.join(root, "TransformerEngine", "transformer_engine", "pytorch", "custom_recipes")
    for name in ("transformer_engine", "transformer_engine.pytorch",
                 "transformer_engine.pytorch.custom_recipes",
                 "transformer_engine.pytorch.quantized_tensor"):
        if name not in sys.modules:
            m = types.ModuleType(name)
            m.__path__ = []
            sys.modules[name] = m
    qt = sys.modules["transformer_engine.pytorch.quantized_tensor"]

    class QuantizedTensorStorage:  # empty base, as the emulation only subclasses it
        pass

    class Quantizer:
        def __init__(self, rowwise: bool = True, columnwise: bool = True):
            self.rowwise_usage = rowwise
            self.columnwise_usage = columnwise

    qt.QuantizedTensorStorage = QuantizedTensorStorage
    qt.Quantizer = Quantizer
    mods = {}
    for short in ("utils", "quantization", "quantization_nvfp4", "quantization_mxfp4"):
        full = f"transformer_engine.pytorch.custom_recipes.{short}"
        spec = importlib.util.spec_from_file_location(full, os.path.join(base, short + ".py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[full] = mod
        setattr(sys.modules["transformer_engine.pytorch.custom_recipes"], short, mod)
        spec.loader.exec_module(mod)
        mods[short] = mod
    return mods


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().astype(np.uint16)


def make_inputs(M, K, N, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    cols = torch.randperm(K, generator=g)[: max(1, K // 1000)]
    x[:, cols] *= 20.0
    w = 0.02 * torch.randn(N, K, generator=g)
    return x.to(torch.bfloat16), w.to(torch.bfloat16)


def load_function_source(path: str, name: str, namespace: dict):
    """Executes one top-level function definition of a reference module (the module as a whole imports packages
    that are not installed here) and returns it."""
    import ast
    with open(path) as f:
        tree = ast.parse(f.read())
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name == name:
            mod = ast.Module(body=[node], type_ignores=[])
            exec(compile(mod, path, "exec"), namespace)
            return namespace[name]
    raise RuntimeError(f"{name} not found in {path}")


def make_rmsnorm_bwd_golden(root: str):
    """RMSNorm backward of the FFN block through the reference's own PyTorch formula
    (low_bits_training/quantization/fused_te_linear.py, _te_ffn_rmsnorm_backward_reference)."""
    fn = load_function_source(os.path.join(root, "low_bits_training", "quantization", "fused_te_linear.py"),
                              "_te_ffn_rmsnorm_backward_reference", {"torch": torch})
    g = torch.Generator().manual_seed(77)
    M, K = 160, 512
    x = torch.randn(M, K, generator=g)
    x[:, torch.randperm(K, generator=g)[:2]] *= 20.0
    x = x.to(torch.bfloat16)
    dy = (1e-3 * torch.randn(M, K, generator=g)).to(torch.bfloat16)
    gamma = (1.0 + 0.1 * torch.randn(K, generator=g)).to(torch.bfloat16)
    inv_rms = torch.rsqrt(x.float().pow(2).mean(dim=1) + 1e-5)
    dx, dgamma = fn(dy, x, gamma, inv_rms)
    out = {"x_bits": bf16_bits(x), "dy_bits": bf16_bits(dy), "gamma_bits": bf16_bits(gamma), "inv_rms": inv_rms.numpy(),
           "dx_bits": bf16_bits(dx), "dgamma": dgamma.numpy()}
    path = os.path.join(HERE, "rmsnorm_bwd_reference_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, {k: v.shape for k, v in out.items()})


def make_scale_swizzle_golden(root: str):
    """The 512-byte scale tile layout through the reference's own torch helper (scale_swizzle in
    fp4_runtime/TK_quantisation/mxfp4_v1/test_mxfp4_quantize.py): distinct bytes in, swizzled tiles out."""
    fn = load_function_source(os.path.join(root, "fp4_runtime", "TK_quantisation", "mxfp4_v1", "test_mxfp4_quantize.py"),
                              "scale_swizzle", {"torch": torch})
    g = torch.Generator().manual_seed(5)
    logical = torch.randint(0, 256, (384, 12), generator=g, dtype=torch.int64).to(torch.uint8)   # 3 x 3 tiles
    out = {"logical": logical.numpy(), "swizzled": fn(logical).numpy()}
    path = os.path.join(HERE, "scale_swizzle_reference_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, {k: v.shape for k, v in out.items()})


def make_mxfp4_golden(root: str):
    """MXFP4 (32-element blocks, E8M0 scales, no tensor scale) through the reference's CPU emulation
    MXFP4QuantizerRef (custom_recipes/quantization_mxfp4.py), decode-centric, and its block-wise qgemm with the
    1/36 factor.  The emulation rounds the scale exponent in the log domain (round(log2(amax))); the CUDA kernels'
    RTE mode rounds the mantissa: the two agree except for block maxima in [sqrt(2), 1.5) x 2^k."""
    mods = load_reference(root)
    qm, utils, quantization = mods["quantization_mxfp4"], mods["utils"], mods["quantization"]
    M, K, N = 256, 512, 128
    x, w = make_inputs(M, K, N, 4242)
    q = qm.MXFP4QuantizerRef(dtype=utils.Fp4Formats.E2M1, rowwise=True, columnwise=True, quant_tile_shape=(1, 32),
                             use_global_scale=False, encode_centric=False)
    qx, qw = q.quantize(x), q.quantize(w)
    y = q.qgemm(qx.data, qw.data, quantization.MMParams(), torch.float32, qx.scale, qw.scale)
    out = {"x_bits": bf16_bits(x), "w_bits": bf16_bits(w),
           "x_data": qx.data.numpy(), "x_scale": qx.scale.view(torch.uint8).numpy(),
           "x_data_t": qx.data_t.numpy(), "x_scale_t": qx.scale_t.view(torch.uint8).numpy(),
           "w_data": qw.data.numpy(), "w_scale": qw.scale.view(torch.uint8).numpy(), "qgemm_f32": y.numpy()}
    path = os.path.join(HERE, "mxfp4_reference_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, {k: v.shape for k, v in out.items()})


def make_tk_gemm_quantize_golden(root: str):
    """The GEMM module's own tile quantiser through the torch reference of its test script
    (torch_nvfp4_quantize and scale_swizzle in ThunderKittens/kernels/gemm/nvfp4_b200/test_quantize.py).  That
    reference calls the module's fp32 -> packed E2M1 cast for its last step; the reference's CPU emulation of the
    same cast (cast_to_fp4x2 of custom_recipes/quantization_nvfp4.py) stands in for it here."""
    mods = load_reference(root)
    cast = mods["quantization_nvfp4"].cast_to_fp4x2
    path = os.path.join(root, "fp4_runtime", "ThunderKittens", "kernels", "gemm", "nvfp4_b200", "test_quantize.py")
    ns = {"torch": torch, "fp32_to_fp4x2": lambda v: cast(v.clamp(-6.0, 6.0))}
    quant = load_function_source(path, "torch_nvfp4_quantize", ns)
    swz = load_function_source(path, "scale_swizzle", ns)
    x, _ = make_inputs(256, 512, 128, 99)
    out = {"a_bits": bf16_bits(x)}
    for scale_2d in (False, True):
        fp4, sc, sg = quant(x, scale_2d)
        tag = "2d" if scale_2d else "1d"
        out[f"{tag}_fp4"] = fp4.numpy()
        out[f"{tag}_sc"] = sc.view(torch.uint8).numpy()
        out[f"{tag}_sc_swizzled"] = swz(sc).view(torch.uint8).numpy()
        out[f"{tag}_sg"] = sg.numpy()
    p = os.path.join(HERE, "tk_gemm_quantize_reference_golden.npz")
    np.savez_compressed(p, **out)
    print("wrote", p, {k: v.shape for k, v in out.items()})


def make_rht_and_norm_golden(root: str):
    """The 16-point Hadamard transform of the reference's CPU emulation (NVFP4QuantizerRef._apply_rht, with and
    without its fixed sign vector) and the forward RMSNorm of the FFN block in the reference's PyTorch formula
    (_te_ffn_rmsnorm_forward_reference in fused_te_linear.py)."""
    mods = load_reference(root)
    qn, utils = mods["quantization_nvfp4"], mods["utils"]
    x, _ = make_inputs(64, 256, 16, 31)
    out = {"x_bits": bf16_bits(x)}
    for sign in (False, True):
        q = qn.NVFP4QuantizerRef(dtype=utils.Fp4Formats.E2M1, rowwise=True, columnwise=True, quant_tile_shape=(1, 16),
                                 with_rht=True, with_random_sign_mask=sign)
        out["rht_signed_bits" if sign else "rht_plain_bits"] = bf16_bits(q._apply_rht(x))
    fwd = load_function_source(os.path.join(root, "low_bits_training", "quantization", "fused_te_linear.py"),
                               "_te_ffn_rmsnorm_forward_reference", {"torch": torch})
    g = torch.Generator().manual_seed(32)
    gamma = (1.0 + 0.1 * torch.randn(256, generator=g)).to(torch.bfloat16)
    normed, inv_rms = fwd(x, gamma, 1e-5)
    out["gamma_bits"] = bf16_bits(gamma)
    out["normed_bits"] = bf16_bits(normed)
    out["inv_rms"] = inv_rms.squeeze(-1).numpy()
    path = os.path.join(HERE, "rht_and_norm_reference_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, {k: v.shape for k, v in out.items()})


def make_sr_state_golden(root: str):
    """A scripted life of the reference's MXFP4SRState (low_bits_training/quantization/mxfp4_sr_state.py) on one
    rank of a world of one and as rank 1 of a declared world of two (no process group: local rows only): the pairs
    handed out by reserve(), and the checkpoint of the single-rank run."""
    import importlib.util
    import json
    path = os.path.join(root, "low_bits_training", "quantization", "mxfp4_sr_state.py")
    spec = importlib.util.spec_from_file_location("ref_mxfp4_sr_state", path)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    names = ["layers.3.ffn", "layers.0.attn", "layers.0.ffn"]
    keys = [ref.ffn_deriv_grad_key(names[0]), ref.qkv_grad_key(names[1]), ref.wo_grad_key(names[1]),
            ref.ffn_w2_grad_key(names[2]), ref.linear_grad_key("head")]
    script = [0, 1, 1, 4, 2, 0, 3, 1]   # indices into keys, in call order
    seed, base = (1 << 64) - 3, 5 << 32
    out = {"names": names, "keys": keys, "script": script, "seed": seed, "subsequence_base": base, "runs": {}}
    for label, rank, world in (("single", 0, 1), ("rank1_of_2", 1, 2)):
        st = ref.MXFP4SRState(keys, device="cpu", user_seed=seed, user_subsequence_base=base, training_steps=10,
                              gradient_accumulation_steps=2, rank=rank, world_size=world)
        pairs = [list(st.reserve(keys[i])) for i in script]
        run = {"reserved": pairs, "peek": [list(st.peek(k)) for k in keys], "local_rows": st._local_state_matrix().tolist(),
               "reservations_per_slot": st.reservations_per_slot, "sorted_keys": list(st.logical_keys)}
        if world == 1:
            sd = st.state_dict()
            run["state_dict"] = {k: (v.tolist() if torch.is_tensor(v) else v) for k, v in sd.items()}
        out["runs"][label] = run
    dst = os.path.join(HERE, "mxfp4_sr_state_reference_golden.json")
    with open(dst, "w") as f:
        json.dump(out, f, indent=1)
    print("wrote", dst)


def make_localcta_sr_state_golden(root: str):
    """A scripted life of the reference's LocalCTASRState (low_bits_training/quantization/localcta_sr_state.py) on
    CPU tensors: rows after a list of advances (the consumer's ``state[1] += 2**32``, done by hand), the checkpoint of
    the single-rank run, the rows after a v1 migration as rank 0 and rank 1 of two, the enable policy over a list of
    environments, and the keys discovered on stand-in modules."""
    import importlib.util
    import json
    path = os.path.join(root, "low_bits_training", "quantization", "localcta_sr_state.py")
    spec = importlib.util.spec_from_file_location("ref_localcta_sr_state", path)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    names = ["layers.3.ffn", "layers.0.attn", "layers.0.ffn"]
    keys = [ref.ffn_deriv_grad_key(names[0]), ref.qkv_grad_key(names[1]), ref.wo_grad_key(names[1]),
            ref.ffn_w2_grad_key(names[2])]
    script = [[0, 1], [1, 2], [1, 1], [3, 1], [2, 3], [0, 1]]   # (index into keys, launches reserved)
    seed, base = (1 << 64) - 2, 7 << 32
    out = {"names": names, "keys": keys, "script": script, "seed": seed, "subsequence_base": base, "runs": {}}
    for label, rank, world in (("single", 0, 1), ("rank1_of_2", 1, 2)):
        st = ref.LocalCTASRState(keys, device="cpu", user_seed=seed, user_subsequence_base=base, training_steps=10,
                                 gradient_accumulation_steps=2, rank=rank, world_size=world)
        run = {"initial_rows": st._local_state_matrix().tolist(), "reservations_per_slot": st.reservations_per_slot,
               "sorted_keys": list(st.logical_keys)}
        for i, n in script:
            st.get(keys[i])[1] += n * ref.SUBSEQUENCE_STRIDE
        run["rows_after_script"] = st._local_state_matrix().tolist()
        if world == 1:
            sd = st.state_dict()
            run["state_dict"] = {k: (v.tolist() if torch.is_tensor(v) else v) for k, v in sd.items()}
        out["runs"][label] = run
    # a v1 table (one per checkpoint, seeds base + slot + 1) taken in by rank 0 and rank 1 of a world of two
    n = len(keys)
    v1_seed_base = 1000
    v1 = {"version": [1], "subsequence_stride": [ref.SUBSEQUENCE_STRIDE], "logical_keys": sorted(keys),
          "states": [[v1_seed_base + s + 1, (3 + s) << 32] for s in range(n)]}
    out["v1"] = {"state_dict": v1, "rows": {}}
    for rank in (0, 1):
        st = ref.LocalCTASRState(keys, device="cpu", user_seed=seed, user_subsequence_base=base, training_steps=10,
                                 gradient_accumulation_steps=2, rank=rank, world_size=2)
        st.migrate_from_v1_state_dict({"version": torch.tensor(v1["version"]), "logical_keys": v1["logical_keys"],
                                       "subsequence_stride": torch.tensor(v1["subsequence_stride"]),
                                       "states": torch.tensor(v1["states"], dtype=torch.int64)})
        out["v1"]["rows"][str(rank)] = st._local_state_matrix().tolist()
    # enable policy
    names_env = ["USE_TK_LOCALCTA", "USE_TK_LOCALCTA_VARIANT", "NVFP4_USE_STOCHASTIC_ROUNDING", "NVFP4_SR_GRAD",
                 "NVFP4_GRAD_SR_AXES", "NVFP4_USE_SCALE_STOCHASTIC_ROUNDING", "NVFP4_SCALE_SR_GRAD", "NVFP4_SR_ACTIVATION",
                 "NVFP4_SCALE_SR_ACTIVATION"]
    envs = [{}, {"USE_TK_LOCALCTA": "1"}, {"USE_TK_LOCALCTA": "1", "USE_TK_LOCALCTA_VARIANT": "V4"},
            {"USE_TK_LOCALCTA": "1", "USE_TK_LOCALCTA_VARIANT": "v4", "NVFP4_USE_STOCHASTIC_ROUNDING": "1"},
            {"USE_TK_LOCALCTA": "1", "USE_TK_LOCALCTA_VARIANT": "v4", "NVFP4_USE_STOCHASTIC_ROUNDING": "1",
             "NVFP4_GRAD_SR_AXES": "none"},
            {"USE_TK_LOCALCTA": "1", "USE_TK_LOCALCTA_VARIANT": "v4", "NVFP4_USE_STOCHASTIC_ROUNDING": "1",
             "NVFP4_SR_GRAD": "0"},
            {"USE_TK_LOCALCTA": "1", "USE_TK_LOCALCTA_VARIANT": "v4", "NVFP4_SR_GRAD": "true", "NVFP4_GRAD_SR_AXES": "col"},
            {"USE_TK_LOCALCTA": "yes", "USE_TK_LOCALCTA_VARIANT": "v4", "NVFP4_USE_SCALE_STOCHASTIC_ROUNDING": "1"},
            {"USE_TK_LOCALCTA": "1", "USE_TK_LOCALCTA_VARIANT": "v4", "NVFP4_USE_SCALE_STOCHASTIC_ROUNDING": "1",
             "NVFP4_SR_GRAD": "0"},
            {"USE_TK_LOCALCTA": "1", "USE_TK_LOCALCTA_VARIANT": "v4", "NVFP4_USE_SCALE_STOCHASTIC_ROUNDING": "1",
             "NVFP4_SR_GRAD": "1", "NVFP4_GRAD_SR_AXES": "off"},
            {"USE_TK_LOCALCTA": "1", "USE_TK_LOCALCTA_VARIANT": "v4", "NVFP4_SCALE_SR_GRAD": "1"},
            {"USE_TK_LOCALCTA": "1", "USE_TK_LOCALCTA_VARIANT": "v4", "NVFP4_SCALE_SR_GRAD": "off",
             "NVFP4_USE_SCALE_STOCHASTIC_ROUNDING": "1"},
            {"USE_TK_LOCALCTA": "off", "USE_TK_LOCALCTA_VARIANT": "v4", "NVFP4_SR_GRAD": "1"},
            {"USE_TK_LOCALCTA": "1", "USE_TK_LOCALCTA_VARIANT": "v4", "NVFP4_SR_ACTIVATION": "1"},
            {"USE_TK_LOCALCTA": "1", "USE_TK_LOCALCTA_VARIANT": "v4", "NVFP4_SCALE_SR_ACTIVATION": "1", "NVFP4_SR_GRAD": "1"}]
    saved = {k: os.environ.pop(k, None) for k in names_env}
    policy = []
    try:
        for env in envs:
            for k in names_env:
                os.environ.pop(k, None)
            os.environ.update(env)
            policy.append({"env": env, "grad_sr": ref.localcta_v4_grad_sr_enabled(),
                           "role": {r: [ref._role_sr_enabled(r), ref._role_scale_sr_enabled(r)]
                                    for r in ("grad", "activation", "weight")}})
    finally:
        for k in names_env:
            os.environ.pop(k, None)
        os.environ.update({k: v for k, v in saved.items() if v is not None})
    out["policy"] = policy
    # discovery on stand-ins that carry the reference's class names
    def stand_in(kind, name):
        m = type(kind, (torch.nn.Module,), {})()
        m._lbt_debug_name = name
        return m
    root_mod = torch.nn.Module()
    root_mod.a = stand_in("FusedAttentionFP4_TK", "layers.0.attention")
    root_mod.b = stand_in("FusedFeedForwardFP4_TK", "layers.0.feed_forward")
    root_mod.c = stand_in("FusedSquaredReLUFeedForwardFP4_TK", "layers.1.feed_forward")
    root_mod.d = torch.nn.Linear(2, 2)
    out["discovered"] = list(ref.discover_logical_keys([root_mod]))
    dst = os.path.join(HERE, "localcta_sr_state_reference_golden.json")
    with open(dst, "w") as f:
        json.dump(out, f, indent=1)
    print("wrote", dst)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the mfu-fp4-training checkout")
    ap.add_argument("--which", default="all", choices=["all", "nvfp4", "rmsnorm_bwd", "scale_swizzle", "mxfp4", "tk_gemm_quantize", "rht_and_norm",
                                                     "sr_state", "localcta_sr_state"])
    args = ap.parse_args()
    if args.which in ("all", "rmsnorm_bwd"):
        make_rmsnorm_bwd_golden(args.reference)
    if args.which in ("all", "scale_swizzle"):
        make_scale_swizzle_golden(args.reference)
    if args.which in ("all", "mxfp4"):
        make_mxfp4_golden(args.reference)
    if args.which in ("all", "tk_gemm_quantize"):
        make_tk_gemm_quantize_golden(args.reference)
    if args.which in ("all", "rht_and_norm"):
        make_rht_and_norm_golden(args.reference)
    if args.which in ("all", "sr_state"):
        make_sr_state_golden(args.reference)
    if args.which in ("all", "localcta_sr_state"):
        make_localcta_sr_state_golden(args.reference)
    if args.which in ("rmsnorm_bwd", "scale_swizzle", "mxfp4", "tk_gemm_quantize", "rht_and_norm", "sr_state",
                      "localcta_sr_state"):
        return
    mods = load_reference(args.reference)
    qn, utils, quantization = mods["quantization_nvfp4"], mods["utils"], mods["quantization"]

    out = {}
    # (1) E2M1 value table / tie rules as pinned by cast_to_fp4x2 / cast_from_fp4x2
    probe = torch.tensor([[-7.0, -6.0, -5.0, -4.5, -3.5, -3.0, -2.5, -2.0, -1.75, -1.5, -1.25, -1.0,
                           -0.75, -0.5, -0.25, -0.1, 0.0, 0.1, 0.25, 0.5, 0.75, 1.0, 1.25, 1.5, 1.75,
                           2.0, 2.5, 3.0, 3.5, 4.5, 5.0, 5.01, 6.0, 7.0, 0.2500001, 0.7499999]],
                         dtype=torch.float32)
    out["e2m1_probe_in"] = probe.numpy()
    out["e2m1_probe_packed"] = qn.cast_to_fp4x2(probe.clamp(-6, 6)).numpy()
    out["e2m1_lut"] = qn.cast_from_fp4x2(torch.arange(256, dtype=torch.uint8).view(1, -1), torch.float32).numpy()
    out["wgrad_sign_vector"] = qn.get_wgrad_sign_vector().numpy()

    # (2) quantise + qgemm on seeded inputs, decode-centric (the emulation's default) and its
    #     encode-centric branch, 1x16 tiles, plus 16x16 weight tiles.
    for tag, (M, K, N, seed) in {"small": (128, 256, 128, 1234), "mid": (256, 512, 384, 20260903)}.items():
        x, w = make_inputs(M, K, N, seed)
        out[f"{tag}_x_bits"] = bf16_bits(x)
        out[f"{tag}_w_bits"] = bf16_bits(w)
        for ec in (False, True):
            q = qn.NVFP4QuantizerRef(dtype=utils.Fp4Formats.E2M1, rowwise=True, columnwise=True,
                                     quant_tile_shape=(1, 16), encode_centric=ec)
            qx = q.quantize(x)
            qw = q.quantize(w)
            pre = f"{tag}_{'ec' if ec else 'dc'}"
            out[f"{pre}_x_data"] = qx.data.numpy()
            out[f"{pre}_x_scale"] = qx.scale.view(torch.uint8).numpy()
            out[f"{pre}_x_data_t"] = qx.data_t.numpy()
            out[f"{pre}_x_scale_t"] = qx.scale_t.view(torch.uint8).numpy()
            out[f"{pre}_x_amax"] = qx.global_amax_row.numpy()
            out[f"{pre}_w_data"] = qw.data.numpy()
            out[f"{pre}_w_scale"] = qw.scale.view(torch.uint8).numpy()
            out[f"{pre}_w_amax"] = qw.global_amax_row.numpy()
            if not ec:
                y = q.qgemm(qx.data, qw.data, quantization.MMParams(), torch.float32,
                            qx.scale, qw.scale, qresult_x=qx, qresult_w=qw)
                out[f"{pre}_qgemm_f32"] = y.numpy()
                out[f"{pre}_x_deq"] = qx.dequantize(torch.float32).numpy()
        q2 = qn.NVFP4QuantizerRef(dtype=utils.Fp4Formats.E2M1, rowwise=True, columnwise=True,
                                  quant_tile_shape=(16, 16))
        qw2 = q2.quantize(w)
        out[f"{tag}_2d_w_data"] = qw2.data.numpy()
        out[f"{tag}_2d_w_scale"] = qw2.scale.view(torch.uint8).numpy()
        out[f"{tag}_2d_w_data_t"] = qw2.data_t.numpy()
        out[f"{tag}_2d_w_scale_t"] = qw2.scale_t.view(torch.uint8).numpy()

    # (3) exhaustive E4M3 cast table on a sweep of fp32 inputs within the clamp range
    sweep = torch.cat([torch.linspace(0, 448, 20001), torch.logspace(-12, 2.7, 20001),
                       torch.tensor([2.0 ** -10, 2.0 ** -9, 1.5 * 2.0 ** -9, 2.0 ** -6, 464.0, 448.0])]).float()
    sweep = sweep.clamp(max=448.0)
    out["e4m3_sweep_in"] = sweep.numpy()
    out["e4m3_sweep_out"] = sweep.to(torch.float8_e4m3fn).view(torch.uint8).numpy()

    path = os.path.join(HERE, "nvfp4_reference_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
