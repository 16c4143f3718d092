"""Writes the golden fixtures of tests/golden from the REFERENCE's own CUDA kernels.

Run on a GPU box where oracle/_ref/libmmh3_ref.so (the reference's attention kernels compiled from
its sources by oracle/Makefile) is present:

    python tests/golden/make_golden.py [output directory]

For small seeded inputs it records what the reference leaves behind: dense BF16 outputs, the INT8 q
and k with their scales, FP8 V and its scale, the quantized attention's output, and VSA's routes,
route counts and output, and Sol-Attn's block statistics, centred keys, routes, pooled tails and
output (in reference_sol.npz), and the scaled INT8 GEMM's outputs and column maxima (in
reference_int8_gemm.npz). The CPU tests then hold the oracle to these files (bit-exact for INT8 and
routes, within the kernels' tolerance for outputs), so the oracle is pinned to the reference itself
even where no GPU is present. Inputs are regenerated from the seeds by the tests.
"""

import ctypes
import pathlib
import sys

import numpy as np
import torch

REPO = pathlib.Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(REPO))
sys.path.insert(0, str(REPO / "tests"))

import gemm_cases  # noqa: E402
import oracle_lib  # noqa: E402
from mmh3_b200 import attention, synthetic  # noqa: E402
from mmh3_b200.vsa import PackedLayout, VsaPlan  # noqa: E402

SCALE = synthetic.softmax_scale()

DENSE_CASES = [(1, 1), (64, 2), (200, 3)]
QUANTIZED_CASES = [(65, 2), (200, 3)]
VSA_CASE = dict(text=70, frames=9, height=16, width=24, audio=40, heads=2, sparsity=0.7)
SOL_CASE = dict(tokens=777, heads=2, tau=0.5, sinks=(0, 1, 2, 3))
# name -> (m, n, k, seed, FP16 output with a bias, SwiGLU)
GEMM_CASES = {"bf16": (130, 384, 256, 41, False, False), "f16_bias": (70, 256, 128, 42, True, False),
              "swiglu": (40, 512, 128, 43, False, True)}


def gemm_operands(name):
    """The operands of a GEMM case as the kernel takes them (SwiGLU rows interleaved)."""
    m, n, k, seed, f16, swiglu = GEMM_CASES[name]
    a, w, a_scales, w_scales, bias = gemm_cases.operands(m, n, k, seed, bias=f16 or swiglu,
                                                          swiglu=swiglu)
    if swiglu:
        w, w_scales, bias = (gemm_cases.interleave(rows) for rows in (w, w_scales, bias))
    return a, w, a_scales, w_scales, bias


def sol_inputs(oracle, tokens, heads):
    """Every block of 64 tokens shares a random direction, so routing is selective."""
    inner = heads * 128
    blocks = -(-tokens // 64)
    directions, state = oracle_lib.lcg(oracle, tokens, blocks * 3 * inner, -1.0, 1.0)
    noise, state = oracle_lib.lcg(oracle, state, tokens * 3 * inner, -1.0, 1.0)
    qkv = directions.reshape(blocks, 3 * inner)[np.arange(tokens) // 64] + \
        noise.reshape(tokens, 3 * inner)
    return synthetic.to_bf16_bits(qkv.reshape(-1)).reshape(tokens, 3, heads, 128)


def lcg_qkv(oracle, tokens, heads, seed):
    values, _ = oracle_lib.lcg(oracle, seed, tokens * 3 * heads * 128, -2.0, 2.0)
    return synthetic.to_bf16_bits(values).reshape(tokens, 3, heads, 128)


def vsa_inputs(oracle, plan, tokens, heads):
    inner = heads * 128
    state = tokens + heads
    directions, state = oracle_lib.lcg(oracle, state, plan.tiles * 3 * inner, -1.0, 1.0)
    tile_of = np.zeros(tokens, dtype=np.int64)
    for tile, (start, length) in enumerate(zip(plan.tile_starts, plan.tile_lengths)):
        tile_of[start:start + length] = tile
    noise, state = oracle_lib.lcg(oracle, state, tokens * 3 * inner, -1.0, 1.0)
    qkv = directions.reshape(plan.tiles, 3 * inner)[tile_of] + noise.reshape(tokens, 3 * inner)
    return synthetic.to_bf16_bits(qkv.reshape(-1)).reshape(tokens, 3, heads, 128)


def main():
    out = pathlib.Path(sys.argv[1]) if len(sys.argv) > 1 else REPO / "tests" / "golden"
    out.mkdir(parents=True, exist_ok=True)
    oracle = oracle_lib.load()
    reference = oracle_lib.load_reference()
    if reference is None or not torch.cuda.is_available():
        raise SystemExit("needs a GPU and oracle/_ref/libmmh3_ref.so")
    arrays = {}
    for tokens, heads in DENSE_CASES:
        inner = heads * 128
        bits = lcg_qkv(oracle, tokens, heads, tokens * 31 + heads)
        qkv = synthetic.bf16_tensor(bits, "cuda")
        output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
        base = qkv.data_ptr()
        assert reference.mmh3_attention_bf16(base, base + 2 * inner, base + 4 * inner,
                                             output.data_ptr(), tokens, heads, 3 * inner, 3 * inner,
                                             3 * inner, inner, SCALE, None) == 0
        torch.cuda.synchronize()
        arrays[f"dense_{tokens}_{heads}"] = output.view(torch.int16).cpu().numpy().view(np.uint16)
    for tokens, heads in QUANTIZED_CASES:
        inner = heads * 128
        bits = lcg_qkv(oracle, tokens, heads, tokens * 17 + heads)
        qkv = synthetic.bf16_tensor(bits, "cuda")
        output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
        workspace = attention.QuantizedWorkspace(tokens, heads)
        layout = attention.qkv_layout(heads)
        raw = workspace.raw()
        base = qkv.data_ptr()
        assert reference.mmh3_attention_quantized(
            base, base + 2 * inner, base + 4 * inner, output.data_ptr(), tokens, heads,
            ctypes.byref(layout), SCALE, None, ctypes.byref(raw), 0, None) == 0
        torch.cuda.synchronize()
        key = f"quantized_{tokens}_{heads}"
        for name in ("query", "key", "value", "query_scales", "key_scales", "value_scales",
                     "value_maxima"):
            arrays[f"{key}_{name}"] = getattr(workspace, name).cpu().numpy()
        arrays[f"{key}_output"] = output.view(torch.int16).cpu().numpy().view(np.uint16)
    case = VSA_CASE
    layout = PackedLayout.text_to_video(case["text"], case["frames"], case["height"],
                                        case["width"], case["audio"])
    plan = VsaPlan.for_layout(layout)
    tokens, heads = len(layout), case["heads"]
    inner = heads * 128
    kept = plan.kept_video_tiles(case["sparsity"])
    bits = vsa_inputs(oracle, plan, tokens, heads)
    qkv = synthetic.bf16_tensor(bits, "cuda")
    output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    workspace = attention.VsaWorkspace(plan, tokens, heads)
    vsa_layout = attention.qkv_layout(heads)
    raw = workspace.raw()
    base = qkv.data_ptr()
    assert reference.mmh3_vsa_attention(
        base, base + 2 * inner, base + 4 * inner, None, inner, output.data_ptr(), tokens, heads,
        ctypes.byref(vsa_layout), SCALE, plan.tiles, plan.prefix_tiles, kept, ctypes.byref(raw),
        None, 0, None) == 0
    torch.cuda.synchronize()
    routes, counts = workspace.routes_host()
    # Only the used prefix of each route row is defined.
    packed = np.concatenate([routes[head, tile, :counts[head, tile]]
                             for head in range(heads) for tile in range(plan.tiles)])
    arrays["vsa_routes"] = packed
    arrays["vsa_route_counts"] = counts
    arrays["vsa_pooled_query"] = workspace.pooled_query.cpu().numpy()
    arrays["vsa_pooled_key"] = workspace.pooled_key.cpu().numpy()
    arrays["vsa_pooled_value"] = workspace.pooled_value.cpu().numpy()
    arrays["vsa_output"] = output.view(torch.int16).cpu().numpy().view(np.uint16)
    np.savez_compressed(out / "reference_kernels.npz", **arrays)
    print("wrote", out / "reference_kernels.npz", sum(a.nbytes for a in arrays.values()), "bytes")

    case = SOL_CASE
    tokens, heads = case["tokens"], case["heads"]
    inner = heads * 128
    bits = sol_inputs(oracle, tokens, heads)
    qkv = synthetic.bf16_tensor(bits, "cuda")
    output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    workspace = attention.SparseWorkspace(tokens, heads)
    sol_layout = attention.qkv_layout(heads)
    raw = workspace.raw()
    base = qkv.data_ptr()
    assert reference.mmh3_sparse_attention(
        base, base + 2 * inner, base + 4 * inner, output.data_ptr(), tokens, heads,
        ctypes.byref(sol_layout), SCALE, case["tau"], *case["sinks"], ctypes.byref(raw), None, 0,
        None) == 0
    torch.cuda.synchronize()
    routes, counts = workspace.routes_host()
    sol = {"routes": np.concatenate([routes[head, block, :counts[head, block]]
                                     for head in range(heads)
                                     for block in range(workspace.blocks)]),
           "route_counts": counts,
           "output": output.view(torch.int16).cpu().numpy().view(np.uint16)}
    for name in ("centroids", "block_keys", "value_sums", "key_mean", "key_variance", "tail_max",
                 "tail_sum", "tail_values", "row_offsets"):
        sol[name] = getattr(workspace, name).cpu().numpy()
    np.savez_compressed(out / "reference_sol.npz", **sol)
    print("wrote", out / "reference_sol.npz", sum(a.nbytes for a in sol.values()), "bytes")

    gemm = {}
    for name, (m, n, k, _, f16, swiglu) in GEMM_CASES.items():
        operands = [None if array is None else torch.from_numpy(np.ascontiguousarray(array)).cuda()
                    for array in gemm_operands(name)]
        pointers = [ctypes.c_void_p(0 if tensor is None else tensor.data_ptr())
                    for tensor in operands]
        result = torch.zeros((m, n // 2 if swiglu else n), dtype=torch.int16, device="cuda")
        tracked = not f16 and not swiglu
        maxima = torch.zeros(max((n - 128) // 128, 1), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        assert reference.mmh3_int8_gemm(
            0, 8, *pointers, ctypes.c_void_p(result.data_ptr()), int(f16), int(swiglu), m, n, k, 0,
            None, None, 0, 0, 0.0, ctypes.c_void_p(maxima.data_ptr() if tracked else 0), 128,
            None) == 0
        torch.cuda.synchronize()
        gemm[f"{name}_output"] = result.cpu().numpy().view(np.uint16)
        if tracked:
            gemm[f"{name}_maxima"] = maxima.cpu().numpy()
    np.savez_compressed(out / "reference_int8_gemm.npz", **gemm)
    print("wrote", out / "reference_int8_gemm.npz", sum(a.nbytes for a in gemm.values()), "bytes")


if __name__ == "__main__":
    main()
