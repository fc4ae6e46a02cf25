"""Wall-clock time of IRuntime::EnqueueWorkload for ResNet-50 int8 through the unmodified Arm NN runtime with the
B200Acc plugin (needs oracle/_ref and the plugin built, and a GPU): buffers copied by the core, imported on every call
(INetworkProperties{Malloc, Malloc}), and pre-imported (IRuntime::ImportInputs / ImportOutputs).

    python tests/plugin_timing.py [batch]
"""
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import hostnet                                    # noqa: E402
from armnn_b200 import configs                    # noqa: E402


def main():
    batch = int(sys.argv[1]) if len(sys.argv) > 1 else 256
    net, info = configs.resnet50(batch, 224)
    rng = np.random.default_rng(3)
    x = rng.integers(-128, 128, size=info["input_shape"]).astype(np.int8)
    y = np.zeros(info["output_shape"], np.int8)
    for mode in ("copy", "import", "preimport"):
        n = hostnet.ArmnnNetwork(net, "B200Acc", import_io=(mode == "import"))
        ts = []
        for _ in range(13):
            t0 = time.perf_counter()
            n.run_into({0: x}, {0: y}, preimported=(mode == "preimport"))
            ts.append(time.perf_counter() - t0)
        ts = sorted(ts[3:])
        print("Arm NN runtime + B200Acc plugin, ResNet-50 batch %d, %-9s: best %.3f ms, median %.3f ms -> %.0f images/s" % (
            batch, mode, ts[0] * 1e3, ts[5] * 1e3, batch / ts[5]))
        n.close()


if __name__ == "__main__":
    main()
