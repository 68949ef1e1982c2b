"""A small, self-ending workload for profiler captures of the streaming kernel:

    python -m qpack_b200.profile_case ROWS [CLUSTER] [CALLS] [THREADS]

ROWS rows of the serving batch (V = 151936; 296 rows = 180 MB, larger than L2 but a fraction of a second of work),
CALLS sample calls (default 3: two warm-ups and the one to capture), THREADS per CTA (128 or 256; default 0 = as
the library chooses for ROWS: 128 above 592 rows).
"""
import sys

import torch

from qpack_b200 import synth
from qpack_b200.sampler import BatchSampler


def main():
    rows = int(sys.argv[1]) if len(sys.argv) > 1 else 296
    cluster = int(sys.argv[2]) if len(sys.argv) > 2 else 0
    calls = int(sys.argv[3]) if len(sys.argv) > 3 else 3
    threads = int(sys.argv[4]) if len(sys.argv) > 4 else 0
    wl = synth.serving_batch(rows=rows)
    x = torch.from_numpy(wl.logits).cuda()
    h = torch.from_numpy(wl.history).cuda()
    bs = BatchSampler(rows, 0)
    bs.set_params(wl.params)
    bs.set_cluster(cluster)
    bs.set_stream_config(threads, 0)
    for _ in range(calls):
        out = bs.sample(x, h)
    bs.check()
    print(out[:4].cpu().numpy())
    bs.close()


if __name__ == "__main__":
    main()
