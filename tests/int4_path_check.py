"""Run by test_int4_paths_gpu.py in a child process with AB_INT4_PATH set: the int4 launcher reads
that variable once per process, so every kernel variant gets a process of its own.  Prints one
line per shape: the kernel the launcher reports and the relative error against the oracle."""
import sys

import numpy as np
import torch

sys.path.insert(0, __file__.rsplit("/", 2)[0])
sys.path.insert(0, __file__.rsplit("/", 1)[0])
import oracle as orc  # noqa: E402
from accel_b200 import runtime  # noqa: E402
from accel_b200 import tensor as T  # noqa: E402
from util import normal, rel_err  # noqa: E402

DEV = "cuda:0"


def main():
    shapes = [tuple(int(v) for v in s.split("x")) for s in sys.argv[1:]]
    for M, K, N in shapes:
        w = normal(2, (K, N), 0.02)
        # constant groups (scale 0, the value carried by the zero point): row 3's first group and,
        # where the row has more than one group, the last group of the last row
        w.reshape(-1)[3 * N:3 * N + 128] = 0.25
        w.reshape(-1)[K * N - 128:] = -0.125
        p, s, z = orc.int4_quantize(w)
        a = normal(1, (M, K))
        want = orc.quant_matmul_int4(a, p, s, z, M, N, K) if M > 1 else \
            orc.quant_matvec_int4(a[0], p, s, z, N, K)[None, :]
        q = T.Int4(torch.from_numpy(p.view(np.int32)).to(DEV), torch.from_numpy(s.view(np.float16)).to(DEV),
                   torch.from_numpy(z.view(np.float16)).to(DEV), K * N)
        x = torch.from_numpy(a).to(DEV)
        got = (T.int4_matmul(x, q) if M > 1 else T.int4_matvec(x[0], q)[None, :]).cpu().numpy()
        print(f"{M}x{K}x{N}\t{rel_err(got, want):.3e}\t{runtime.last_selection()}", flush=True)


if __name__ == "__main__":
    main()
