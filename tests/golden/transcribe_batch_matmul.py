"""Transcribes the BatchMatMul known-answer vectors of the Arm NN reference's layer tests into ref_layer_tests.json.

    python tests/golden/transcribe_batch_matmul.py <arm nn source tree>

Reads src/backends/backendsCommon/test/layerTests/BatchMatMulTestImpl.cpp as text (nothing of the reference is built or
run) and, for each test that RefLayerTests.cpp instantiates for QAsymmS8 with plain (batch, row, column) operands,
records the descriptor's transpose flags, the operand shapes and the three value lists.  All of these tests use
scale 1.0 / offset 0, so the listed real values are the quantised values.
"""
import json
import os
import re
import sys

TESTS = ["BatchMatMul2DSimpleTest", "BatchMatMul3DSimpleTest", "BatchMatMul3DBatchTest", "BatchMatMul3DBroadcastTest",
         "BatchMatMul3D2DBroadcastTest", "BatchMatMul2DTinyTest", "BatchMatMul3DNonSquareTest", "BatchMatMul2DTranspSimpleTest"]


def numbers(text):
    return [int(float(v)) for v in re.findall(r"-?\d+(?:\.\d+)?", text)]


def main(root):
    path = os.path.join(root, "src/backends/backendsCommon/test/layerTests/BatchMatMulTestImpl.cpp")
    lines = open(path).read().split("\n")
    src = "\n".join(lines)
    here = os.path.dirname(os.path.abspath(__file__))
    out_path = os.path.join(here, "ref_layer_tests.json")
    golden = json.load(open(out_path))
    for name in TESTS:
        m = re.search(r"LayerTestResult<T, \d> %s\(" % name, src)
        start = m.start()
        end = src.index("return BatchMatMulTestImpl", start)
        body = src[start:end]
        line0 = src[:start].count("\n") + 1
        desc = re.search(r"armnn::BatchMatMulDescriptor\(([^)]*)\)", body)
        flags = [f.strip() == "true" for f in desc.group(1).split(",")] if desc and desc.group(1).strip() else []
        flags += [False] * (4 - len(flags))           # (transposeX, transposeY, adjointX, adjointY)
        assert not flags[2] and not flags[3]
        scale = float(re.search(r"float qScale = ([0-9.]+)f", body).group(1))
        offset = int(re.search(r"int32_t qOffset = (-?\d+)", body).group(1))
        assert scale == 1.0 and offset == 0
        shapes = {k: numbers(re.search(r"armnn::TensorInfo %s\(\{([^}]*)\}" % k, body).group(1))
                  for k in ("inputXInfo", "inputYInfo", "outputInfo")}
        vals = {k: numbers(re.search(r"std::vector<T> %s = armnnUtils::QuantizedVector<T>\(\{([^}]*)\}" % k, body, re.S).group(1))
                for k in ("inputX", "inputY", "outputExpected")}
        golden["batch_matmul_" + name[len("BatchMatMul"):-len("Test")]] = {
            "source": "BatchMatMulTestImpl.cpp:%d %s<QAsymmS8> (RefLayerTests.cpp:1057-1129)" % (line0, name),
            "transpose_x": flags[0], "transpose_y": flags[1],
            "x_shape": shapes["inputXInfo"], "y_shape": shapes["inputYInfo"], "out_shape": shapes["outputInfo"],
            "scale": scale, "zp": offset, "x": vals["inputX"], "y": vals["inputY"], "out": vals["outputExpected"], "tolerance": 1}
    json.dump(golden, open(out_path, "w"), indent=1)
    print("wrote", out_path)


if __name__ == "__main__":
    main(sys.argv[1])
