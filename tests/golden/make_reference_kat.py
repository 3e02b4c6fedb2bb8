"""Writes tests/golden/reference_kat.json: the known-answer vectors that Neureka's own test-suite holds for
the convolution / broadcast / elementwise path, transcribed by hand from the reference's test sources
(the reference is a JVM library and cannot be executed where this repository is built, so the vectors are
copied as text; every entry cites the file and lines it was read from, relative to the reference root).

    python tests/golden/make_reference_kat.py
"""
import json
import os

T = "src/test/groovy"
KAT = {
    # ---- forward "x" -----------------------------------------------------------------------------------
    "conv_forward": [
        {"src": f"{T}/ut/tensors/Tensor_Convolution_Spec.groovy:52-82", "a_shape": [3, 3], "a": [1, 2, 3, 4, 5, 6, 7, 8, 9],
         "b_shape": [2, 2], "b": [1, 2, 0, -1], "out_shape": [2, 2], "out": [0, 2, 6, 8]},
        {"src": f"{T}/ut/tensors/Tensor_Convolution_Spec.groovy:85-110", "a_shape": [2, 2], "a": [1, 3, 6, -8],
         "b_shape": [2, 2], "b": [-2, 1, 4, 5], "out_shape": [1, 1], "out": [-15]},
        {"src": f"{T}/ut/tensors/Tensor_Convolution_Spec.groovy:113-137", "a_shape": [2, 3], "a": [1, 3, 6, -8, 2, 4],
         "b_shape": [1, 2], "b": [-2, 1], "out_shape": [2, 2], "out": [1, 0, 18, 0]},
        {"src": f"{T}/ut/tensors/Tensor_Convolution_Spec.groovy:141-168", "a_shape": [2, 2, 2], "a": [1, 3, 6, -8, 2, 4, 5, 7],
         "b_shape": [1, 2, 2], "b": [-2, 1, 4, 5], "out_shape": [2, 1, 1], "out": [-15, 55]},
        {"src": f"{T}/ut/tensors/Tensor_Convolution_Spec.groovy:170-215", "a_shape": [2, 3, 1], "a": [3, 2, -1, -2, 2, 4],
         "b_shape": [1, 3, 2], "b": [4, -1, 3, 2, 3, -1], "out_shape": [2, 1, 2], "out": [15, 2, 10, 2]},
        {"src": f"{T}/ut/tensors/Tensor_Convolution_Spec.groovy:422-447", "a_shape": [3, 2, 1], "a": [1, 2, 3, 4, 5, 6],
         "b_shape": [1, 2, 3], "b": [1, 2, 3, 4, 5, 6], "out_shape": [3, 1, 3], "out": [9, 12, 15, 19, 26, 33, 29, 40, 51]},
        {"src": f"{T}/st/tests/BroadSystemTest.java:321-340", "a_shape": [4, 1], "a": [-2, -1, 4, 3],
         "b_shape": [1, 3], "b": [2, -4, 3], "out_shape": [4, 3], "out": [-4, 8, -6, -2, 4, -3, 8, -16, 12, 6, -12, 9]},
        {"src": f"{T}/st/tests/BroadSystemTest.java:342-360", "a_shape": [4, 2], "a": [-1, 2, -3, 1, 4, -5, 2, 3],
         "b_shape": [2, 3], "b": [4, -2, 8, -1, -5, 2], "out_shape": [3, 2], "out": [-10, 35, 7, -16, 9, -52]},
        {"src": f"{T}/st/tests/BroadSystemTest.java:362-380", "a_shape": [1, 1], "a": [2],
         "b_shape": [2, 3], "b": [4, -2, 8, -1, -5, 2], "out_shape": [2, 3], "out": [8, -4, 16, -2, -10, 4]},
        {"src": f"{T}/st/tests/BroadSystemTest.java:382-410", "a_shape": [2, 3, 2], "a": [1, 2, 3, 4, 0, 2, 3, 4, 2, -1, -2, -3],
         "b_shape": [2, 2, 3], "b": [-1, 3, 0, 2, -3, 1, 2, -3, 0, 4, 5, -1], "out_shape": [1, 2, 2], "out": [-4, 0, -13, -2]},
        {"src": f"{T}/st/tests/BroadSystemTest.java:19-25 (forward part)", "a_shape": [2, 2], "a": [-1, 2, -3, 3],
         "b_shape": [1, 1], "b": [-3], "out_shape": [2, 2], "out": [3, -6, 9, -9]},
        {"src": f"{T}/st/tests/BroadSystemTest.java:279-299 (forward part)", "a_shape": [2, 2, 1], "a": [1, 2, 2, -3],
         "b_shape": [1, 2, 2], "b": [-2, 3, 1, 2], "out_shape": [2, 1, 2], "out": [0, 7, -7, 0]},
    ],
    # [200,300,1] x [1,300,200] of 2s and 3s -> every element 1800
    "conv_forward_constant": [
        {"src": f"{T}/st/tests/CrossDeviceSystemTest.java:95-103", "a_shape": [200, 300, 1], "a_fill": 2,
         "b_shape": [1, 300, 200], "b_fill": 3, "out_shape": [200, 1, 200], "out_fill": 1800},
    ],
    # identical result for row-major and column-major operands
    "conv_forward_column_major": [
        {"src": f"{T}/ut/tensors/Tensor_Convolution_Spec.groovy:449-465", "a_shape": [3, 2, 1], "a": [1, 2, 3, 4, 5, 6],
         "b_shape": [1, 2, 3], "b": [1, 2, 3, 4, 5, 6], "b_raw_column_major": [1, 4, 2, 5, 3, 6],
         "out_shape": [3, 1, 3], "out": [9, 12, 15, 19, 26, 33, 29, 40, 51]},
    ],
    # conv on a strided slice: a = [4,6] 1..; slice rows 0,2 / cols 1,3 after the documented writes
    "conv_forward_sliced": [
        {"src": f"{T}/it/Cross_Device_Sliced_Tensor_System_Test.groovy:296-336",
         "parent_shape": [4, 6],
         "parent": [1, 1, 3, 2, 5, 6, 7, 8, 8, 1, 2, 3, 4, 8, 8, 4, 8, 9, 1, 2, 3, 4, 5, 6],
         "slice_shape": [2, 2], "slice_offset": [0, 1], "slice_spread": [2, 2], "slice_items": [1, 2, 8, 4],
         "b_shape": [2, 2], "b": [-2, 3, 1, 2], "out": [20]},
    ],
    # ---- XConv ("«x" / "x»") -----------------------------------------------------------------------------
    "xconv": [
        {"src": f"{T}/st/tests/BroadSystemTest.java:232-275 and :412-436", "drain_shape": [2, 3],
         "t1_shape": [5, 2], "t1": [-2, 3, 6, 3, -1, 0, 2, 4, 2, 1],
         "t2_shape": [4, 2], "t2": [1, 2, -3, 2, 4, -2, -1, 5], "out": [-26, 10, 32, 15, 34, 3]},
    ],
    # ---- conv autograd -------------------------------------------------------------------------------------
    "conv_autograd": [
        {"src": f"{T}/st/tests/BroadSystemTest.java:19-27", "a_shape": [2, 2], "a": [-1, 2, -3, 3], "b_shape": [1, 1], "b": [-3],
         "error_shape": [2, 2], "error": [1, 1, 1, 1], "grad_a": [-3, -3, -3, -3]},
        {"src": f"{T}/st/tests/BroadSystemTest.java:279-299; {T}/st/tests/CrossDeviceSystemTest.java:105-125",
         "a_shape": [2, 2, 1], "a": [1, 2, 2, -3], "b_shape": [1, 2, 2], "b": [-2, 3, 1, 2],
         "error_shape": [2, 1, 2], "error": [1, 1, 1, 1], "grad_a": [1, 3, 1, 3]},
    ],
    # two-layer chain: i_a x w_a -> o_a ; o_a x w_b -> o_b ; o_a x w_c -> o_c ; out = o_b*o_c ; backward ones
    "conv_autograd_chain": {
        "src": f"{T}/ut/tensors/Tensor_Convolution_Spec.groovy:303-366",
        "i_a": {"shape": [2, 1], "data": [1, 2]}, "w_a": {"shape": [2, 2], "data": [1, 3, 4, -1]},
        "w_b": {"shape": [2, 2], "data": [-2, 1, 2, -1]}, "w_c": {"shape": [2, 2], "data": [0.5, 3, -2, -0.5]},
        "o_a": [9, 1], "o_b": [-17, 17], "o_c": [7.5, -18.5], "out": [-127.5, -314.5],
        "grad_w_b": [67.5, 7.5, -166.5, -18.5],
        "w_a_after_apply": [-93.5, -30.5, -185.0, -68.0],
    },
    # ---- broadcast -------------------------------------------------------------------------------------------
    "broadcast_forward_mul": [
        {"src": f"{T}/st/tests/BroadSystemTest.java:439-454", "a_shape": [1, 3], "a": [2, -1, 3], "b_shape": [2, 1], "b": [4, -2],
         "out_shape": [2, 3], "out": [8, -4, 12, -4, 2, -6]},
    ],
    "broadcast_backward_mul_both": [
        {"src": f"{T}/st/tests/BroadSystemTest.java:456-487", "origin_shape": [1, 3], "handle_shape": [2, 1], "handle": [2, -1],
         "drain_shape": [2, 3], "drain": [8, -4, -4, 2, 12, -6], "out": [14, -20, -2]},
    ],
    # a = [2,2] 1..4 ; b = 8,9 cyclic in bShape ; c = op(a,b) ; backward error [5,-2,7,3]
    "broadcast_autograd": [
        {"src": f"{T}/ut/tensors/Tensor_Operation_Spec.groovy:421-424", "op": "+", "b_shape": [1], "which_grad": "a", "c": [9, 10, 11, 12], "grad": [5, -2, 7, 3]},
        {"src": f"{T}/ut/tensors/Tensor_Operation_Spec.groovy:426-429", "op": "*", "b_shape": [1], "which_grad": "a", "c": [8, 16, 24, 32], "grad": [40, -16, 56, 24]},
        {"src": f"{T}/ut/tensors/Tensor_Operation_Spec.groovy:431-434", "op": "+", "b_shape": [2, 1], "which_grad": "b", "c": [9, 10, 12, 13], "grad": [3, 10]},
        {"src": f"{T}/ut/tensors/Tensor_Operation_Spec.groovy:436-439", "op": "+", "b_shape": [1], "which_grad": "b", "c": [9, 10, 11, 12], "grad": [13]},
        {"src": f"{T}/ut/tensors/Tensor_Operation_Spec.groovy:441-444", "op": "+", "b_shape": [1, 2], "which_grad": "b", "c": [9, 11, 11, 13], "grad": [12, 1]},
        {"src": f"{T}/ut/tensors/Tensor_Operation_Spec.groovy:446-449", "op": "+", "b_shape": [2], "which_grad": "b", "c": [9, 11, 11, 13], "grad": [12, 1]},
        {"src": f"{T}/ut/tensors/Tensor_Operation_Spec.groovy:451-454", "op": "-", "b_shape": [1, 2], "which_grad": "b", "c": [-7, -7, -5, -5], "grad": [-12, -1]},
        {"src": f"{T}/ut/tensors/Tensor_Operation_Spec.groovy:456-459", "op": "-", "b_shape": [2], "which_grad": "b", "c": [-7, -7, -5, -5], "grad": [-12, -1]},
        {"src": f"{T}/ut/tensors/Tensor_Operation_Spec.groovy:461-464", "op": "rsub", "b_shape": [1, 2], "which_grad": "b", "c": [7, 7, 5, 5], "grad": [12, 1]},
    ],
    # slice addition: a = [11,11] filled cyclically with 3..19 ; x = a[1:-1, :] ; y = a[0:-2, :] ; t = x + y
    "sliced_addition": {
        "src": f"{T}/ut/tensors/Tensor_Operation_Spec.groovy:352-378",
        "first_50": [17, 19, 21, 23, 25, 27, 12, 14, 16, 18, 20, 22, 24, 26, 28, 30, 32, 17, 19, 21, 23, 25, 27, 12, 14, 16, 18,
                     20, 22, 24, 26, 28, 30, 32, 17, 19, 21, 23, 25, 27, 12, 14, 16, 18, 20, 22, 24, 26, 28, 30],
    },
    # ---- elementwise functions ---------------------------------------------------------------------------------
    "tanh_chain": {"src": f"{T}/st/tests/BroadSystemTest.java:29-45", "x": 0.1, "expr": "tanh(i0) then i0*100",
                   "value_4dp": 9.9668, "grad_4dp": 99.0066},
    # ---- views -----------------------------------------------------------------------------------------------------
    "inline_arrays": [
        {"src": f"{T}/it/Cross_Device_Sliced_Tensor_System_Test.groovy:236-240", "parent_shape": [4, 6],
         "slice_shape": [3, 4], "slice_offset": [1, 0], "slice_spread": [1, 1], "inline": [3, 4, 6, 1, 4, 1, 1, 0, 1, 1]},
        {"src": f"{T}/it/Cross_Device_Sliced_Tensor_System_Test.groovy:236-240 (a fresh [3,4] tensor)", "parent_shape": [3, 4],
         "slice_shape": None, "inline": [3, 4, 4, 1, 4, 1, 0, 0, 1, 1]},
    ],
    # ---- MatMul / DotProduct ("next" rows: the callers of the contraction kernels) -----------------------------------------
    "matmul": [
        {"src": f"{T}/ut/backend/Matrix_Multiplication_Spec.groovy:22-35 (andFill repeats 1,2,3 / 2,-4,-1)", "M": 1, "K": 7, "N": 8,
         "a": [1, 2, 3, 1, 2, 3, 1], "b": [2, -4, -1] * 18 + [2, -4], "c": [-22, -10, -7, -22, -10, -7, -22, -10]},
        {"src": f"{T}/ut/backend/Matrix_Multiplication_Spec.groovy:68-75", "M": 2, "K": 2, "N": 2, "a": [4, 3, 2, 1], "b": [-0.5, 1.5, 1, -2], "c": [1, 0, 0, 1]},
        {"src": f"{T}/ut/backend/Matrix_Multiplication_Spec.groovy:69", "M": 1, "K": 2, "N": 1, "a": [-2, 1], "b": [-1, -1.5], "c": [0.5]},
        {"src": f"{T}/ut/backend/Matrix_Multiplication_Spec.groovy:70", "M": 2, "K": 1, "N": 2, "a": [-2, 1], "b": [-1, -1.5], "c": [2.0, 3.0, -1.0, -1.5]},
    ],
    "dot": [
        {"src": f"{T}/ut/tensors/Tensor_Dot_Product_Spec.groovy:29-40", "a": [3, 2], "b": [1, -0.5], "value": 2.0},
        {"src": f"{T}/ut/tensors/Tensor_Dot_Product_Spec.groovy:42-57 (rows of [[1,2],[3,4]])", "a": [1, 2], "b": [3, 4], "value": 11.0},
        {"src": f"{T}/ut/tensors/Tensor_Dot_Product_Spec.groovy:87-103", "a": [-1, -3, 0, 4, 2], "b": [1, 2, 7, -1, 3], "value": -5.0},
        {"src": f"{T}/ut/tensors/Tensor_Dot_Product_Spec.groovy:59-85 (forward 4, error 0.5 -> gradient of w = 0.5 * a)", "a": [4, -1, 2], "b": [1, 0, 0],
         "value": 4.0, "error": 0.5, "grad_b": [2, -0.5, 1]},
    ],
    # ---- RNG ----------------------------------------------------------------------------------------------------------
    "fill_randomly": {
        "src": "src/test/groovy/ut/backend/core/Randomization_Spec.groovy:58-62",
        "seed": 42, "f32": [-0.48528543, -1.4547276], "f64": [-0.485285426832534, -1.454727674701364],
    },
}

if __name__ == "__main__":
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_kat.json")
    with open(out, "w") as f:
        json.dump(KAT, f, indent=1)
    print("wrote", out)
