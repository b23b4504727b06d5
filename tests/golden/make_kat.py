"""Writes tests/golden/numr_kat.json: the known answers numr's own tests hold for the
dense-GEMM path, transcribed as data from the test sources (numr is Rust and cannot be
run here, so the literals are read from the files; each entry names its source).

Run: python tests/golden/make_kat.py
"""
import json
from pathlib import Path

KAT = {
    "i8_matmul": [
        {"src": "tests/backend_parity/matmul/i8_cuda.rs:168-178", "a_shape": [2, 2], "a": [1, 2, 3, 4],
         "b_shape": [2, 2], "b": [5, 6, 7, 8], "out": [19, 22, 43, 50]},
        {"src": "tests/backend_parity/matmul/i8_cuda.rs:186-196", "a_shape": [2, 2], "a": [-1, 2, 3, -4],
         "b_shape": [2, 2], "b": [5, -6, -7, 8], "out": [-19, 22, 43, -50]},
        {"src": "tests/backend_parity/matmul/i8_cuda.rs:209-219", "a_shape": [2, 4],
         "a": [127, 127, 127, 127, -128, -128, -128, -128], "b_shape": [4, 2],
         "b": [127, -128, 127, -128, 127, -128, 127, -128], "out": [64516, -65024, -65024, 65536]},
        {"src": "tests/backend_parity/matmul/i8_cuda.rs:226-236", "a_shape": [2, 3], "a": [1, 2, 3, 4, 5, 6],
         "b_shape": [3, 1], "b": [7, 8, 9], "out": [50, 122]},
        {"src": "tests/backend_parity/matmul/i8_cuda.rs:255-265", "a_shape": [2, 2, 2],
         "a": [1, 2, 3, 4, 5, 6, 7, 8], "b_shape": [2, 2, 2], "b": [1, 0, 0, 1, 2, 0, 0, 2],
         "out": [1, 2, 3, 4, 10, 12, 14, 16]},
    ],
    "i8_matmul_bias": [
        {"src": "src/ops/cpu/matmul_i8.rs:137-147", "a_shape": [2, 2], "a": [1, 2, 3, 4], "b_shape": [2, 2],
         "b": [5, 6, 7, 8], "bias": [1, -2], "out": [20, 20, 44, 48]},
        {"src": "src/ops/cpu/matmul_i8.rs:151-161", "a_shape": [1, 4], "a": [127, 127, 127, 127],
         "b_shape": [4, 1], "b": [127, 127, 127, 127], "bias": [1000], "out": [65516]},
        {"src": "src/ops/cpu/matmul_i8.rs:164-177", "a_shape": [2, 2, 2], "a": [1, 2, 3, 4, 5, 6, 7, 8],
         "b_shape": [2, 2, 2], "b": [1, 0, 0, 1, 2, 0, 0, 2], "bias": [1, -2],
         "out": [2, 0, 4, 2, 11, 10, 15, 14]},
        {"src": "src/runtime/cpu/kernels/simd/matmul/int8.rs:123-140", "a_shape": [1, 1], "a": [12],
         "b_shape": [1, 1], "b": [11], "bias": [5], "out": [137]},
    ],
    # The ragged 20x9 @ 9x5 case has no literal answer in the reference (CPU is its
    # reference); the generator is recorded so the oracle and the GPU replay the same inputs.
    "i8_generated": [
        {"src": "tests/backend_parity/matmul/i8_cuda.rs:243-246", "a_shape": [20, 9], "a_gen": "(i % 61) - 30",
         "b_shape": [9, 5], "b_gen": "(i * 7 % 59) - 29"},
    ],
    "fp8_matmul": [
        {"src": "tests/backend_parity/fp8_matmul.rs:63-79", "a_shape": [2, 3], "a": [1, 2, 3, 4, 5, 6],
         "b_shape": [3, 2], "b": [1, 2, 3, 4, 5, 6], "scale_a": 1.0, "scale_b": 1.0,
         "out": [22, 28, 49, 64], "rtol": 0.1, "atol": 0.5},
        {"src": "tests/backend_parity/fp8_matmul.rs:82-96", "a_shape": [2, 2], "a": [1, 2, 3, 4],
         "b_shape": [2, 2], "b": [1, 2, 3, 4], "scale_a": 2.0, "scale_b": 0.5, "out": [7, 10, 15, 22],
         "rtol": 0.1, "atol": 0.5},
    ],
    # conv_transpose1d known answers of the CPU kernel's own unit tests (groups = 1): x [1, 1, L],
    # w [c_in = 1, c_out = 1, K], padding (left, right)
    "conv_transpose1d": [
        {"src": "src/runtime/cpu/kernels/conv_transpose.rs:150-161", "x": [1, 2, 3], "w": [1, 1, 1], "stride": 1,
         "padding": [0, 0], "output_padding": 0, "dilation": 1, "out": [1, 3, 6, 5, 3]},
        {"src": "src/runtime/cpu/kernels/conv_transpose.rs:163-173", "x": [1, 2], "w": [1, 1, 1], "stride": 2,
         "padding": [0, 0], "output_padding": 0, "dilation": 1, "out": [1, 1, 3, 2, 2]},
        {"src": "src/runtime/cpu/kernels/conv_transpose.rs:177-197", "x": [1, 2, 3], "w": [1, 10, 100], "stride": 2,
         "padding": [1, 1], "output_padding": 0, "dilation": 1, "out": [10, 102, 20, 203, 30]},
    ],
    # inputs of the conv parity tests whose answers follow from their definition (moving sum, box sum)
    "conv_forward": [
        {"src": "tests/backend_parity/conv.rs:18-20 (conv1d moving sum, Valid, stride 1)", "kind": "conv1d",
         "x_shape": [1, 1, 5], "x": [1, 2, 3, 4, 5], "w_shape": [1, 1, 3], "w": [1, 1, 1], "out": [6, 9, 12]},
        {"src": "tests/backend_parity/conv.rs:73-75 (conv2d box sum, Valid, stride 1)", "kind": "conv2d",
         "x_shape": [1, 1, 3, 3], "x": [1, 2, 3, 4, 5, 6, 7, 8, 9], "w_shape": [1, 1, 2, 2], "w": [1, 1, 1, 1],
         "out": [12, 16, 24, 28]},
    ],
    "fp8_e4m3_codec": {
        "src": "src/dtype/fp8.rs:60-76,859-861,1035-1112",
        "constants": {"ZERO": 0x00, "ONE": 0x38, "NEG_ONE": 0xB8, "MAX": 0x7E, "MIN_POSITIVE": 0x08, "NAN": 0x7F},
        "encode_bits": [[0.0, 0x00], [-0.0, 0x80], [1.0, 0x38], [-1.0, 0xB8], [448.0, 0x7E],
                        [0.015625, 0x08]],
        "subnormals_roundtrip": [1, 2, 3, 4, 5, 6, 7],          # m * 2^-9 encodes to bits m
        "flush_to_zero": [2.0 ** -10, 2.0 ** -11, 2.0 ** -20, 1e-10],
        "rounding": [[0.75 * 2.0 ** -9, 2.0 ** -9], [1.5 * 2.0 ** -9, 2.0 * 2.0 ** -9]],
        "exact_normals": [0.5, 1.0, 1.5, 2.0, 3.0, 16.0, 448.0, 0.015625],
        "saturate_to_448": [1e9, float("inf")],
    },
    "fp8_e5m2_codec": {
        "src": "src/dtype/fp8.rs:946-992,1120-1198",
        "encode_bits": [[0.0, 0x00]],
        "subnormals_roundtrip": [1, 2, 3],                      # m * 2^-16 encodes to bits m
        "flush_to_zero": [2.0 ** -17, 2.0 ** -18, 2.0 ** -30, 1e-12],
        "rounding": [[0.75 * 2.0 ** -16, 2.0 ** -16], [1.5 * 2.0 ** -16, 2.0 * 2.0 ** -16]],
        "exact_normals": [0.5, 1.0, 1.5, 2.0, 3.0, 16.0, 57344.0, 0.25],
        "infinity_preserved": [float("inf")],
    },
    "shapes": {
        "src": "src/ops/matmul.rs:266-421",
        "validate_matmul_shapes": [
            {"a": [2, 3], "b": [3, 4], "mkn": [2, 3, 4]},
            {"a": [2, 3], "b": [4, 5], "mkn": None},
            {"a": [3], "b": [3, 4], "mkn": [1, 3, 4]},
            {"a": [2, 3], "b": [3], "mkn": [2, 3, 1]},
        ],
        "matmul_output_shape": [
            {"a": [2, 3], "b": [3, 4], "out": [2, 4]},
            {"a": [5, 2, 3], "b": [5, 3, 4], "out": [5, 2, 4]},
            {"a": [5, 2, 3], "b": [3, 4], "out": [5, 2, 4]},
        ],
        "matmul_bias_shapes": [
            {"a": [2, 3], "b": [4, 5], "bias": [5], "ok": False},
            {"a": [2, 3], "b": [3, 4], "bias": [2, 4], "ok": False},
            {"a": [2, 3], "b": [3, 4], "bias": [3], "ok": False},
            {"a": [2, 3], "b": [3, 4], "bias": [4], "ok": True},
            {"a": [5, 2, 3], "b": [5, 3, 4], "bias": [4], "ok": True},
        ],
        "batch_indices": [
            {"a": [2, 4, 3, 2], "b": [2, 1, 2, 1], "out": [2, 4, 3, 1], "a_idx": [0, 1, 2, 3, 4, 5, 6, 7],
             "b_idx": [0, 0, 0, 0, 1, 1, 1, 1]},
            {"a": [2, 4, 3, 2], "b": [1, 4, 2, 3], "out": [2, 4, 3, 3], "a_idx": [0, 1, 2, 3, 4, 5, 6, 7],
             "b_idx": [0, 1, 2, 3, 0, 1, 2, 3]},
            {"a": [2, 4, 3, 2], "b": [4, 2, 3], "out": [2, 4, 3, 3], "a_idx": [0, 1, 2, 3, 4, 5, 6, 7],
             "b_idx": [0, 1, 2, 3, 0, 1, 2, 3]},
            {"a": [2, 1, 3, 2], "b": [1, 4, 2, 3], "out": [2, 4, 3, 3], "a_idx": [0, 0, 0, 0, 1, 1, 1, 1],
             "b_idx": [0, 1, 2, 3, 0, 1, 2, 3]},
            {"a": [3, 2], "b": [2, 4], "out": [3, 4], "a_idx": [0], "b_idx": [0]},
        ],
        "is_transposed_b": [
            {"shape": [4, 3], "strides": [1, 4], "k": 4, "n": 3, "is": True},
            {"shape": [4, 3], "strides": [3, 1], "k": 4, "n": 3, "is": False},
            {"shape": [4, 3], "strides": [0, 4], "k": 4, "n": 3, "is": False},
            {"shape": [4, 3], "strides": [1, -4], "k": 4, "n": 3, "is": False},
            {"shape": [4, 3], "strides": [-1, 4], "k": 4, "n": 3, "is": False},
            {"shape": [2, 4, 3], "strides": [12, 1, 4], "k": 4, "n": 3, "is": True},
            {"shape": [5, 2, 4, 3], "strides": [24, 12, 1, 4], "k": 4, "n": 3, "is": True},
            {"shape": [2, 4, 3], "strides": [24, 1, 4], "k": 4, "n": 3, "is": False},
            {"shape": [1, 4, 3], "strides": [999, 1, 4], "k": 4, "n": 3, "is": True},
        ],
    },
    "dtype_rules": {
        "src": "src/ops/matmul_dtype.rs:19-100",
        "output_dtype": {"I8": "I32", "F32": "F32", "BF16": "BF16", "F16": "F16"},
        "i8_bias_must_be": "I32",
        "epilogue_rejects": ["I8"],
    },
    "activation_codes": {"src": "src/ops/traits/gemm_epilogue.rs:34-43",
                         "None": 0, "ReLU": 1, "GELU": 2, "SiLU": 3, "Sigmoid": 4, "Tanh": 5},
    "tolerances": {"src": "tests/common/mod.rs:227-237",
                   "F32": [1e-5, 1e-6], "F16": [0.01, 0.1], "BF16": [0.01, 0.1], "FP8E4M3": [0.3, 2.5],
                   "FP8E5M2": [1.0, 2.5]},
}

if __name__ == "__main__":
    out = Path(__file__).with_name("numr_kat.json")
    out.write_text(json.dumps(KAT, indent=1, allow_nan=True) + "\n")
    print(out)
