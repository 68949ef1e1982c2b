"""A small, self-ending workload for profiler captures of the streaming kernel:

    python -m qpack_b200.profile_case ROWS [CLUSTER] [CALLS] [THREADS] [WORKLOAD]

ROWS rows of the serving batch (V = 151936; 296 rows = 180 MB, larger than L2 but a fraction of a second of work),
CALLS sample calls (default 3: two warm-ups and the one to capture), THREADS per CTA (128 or 256; default 0 = as
the library chooses for ROWS: 128 above 592 rows).  WORKLOAD: serving (default; config 4), llama3 (config 2: V =
128256, top_k off, every row on the whole-row kernel) or mixed (config 3: V = 201088, both kernels).  Prints the
device time per call of the last CALLS - 2 calls (CUDA events).
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
    workload = sys.argv[5] if len(sys.argv) > 5 else "serving"
    wl = {"serving": synth.serving_batch, "llama3": synth.llama3_batch, "mixed": synth.mixed_batch}[workload](rows=rows)
    x = torch.from_numpy(wl.logits).cuda()
    h = torch.from_numpy(wl.history).cuda() if wl.history is not None else None
    bs = BatchSampler(rows, 0)
    bs.set_params(wl.params)
    bs.set_cluster(cluster)
    bs.set_stream_config(threads, 0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(calls):
        if i == 2:
            e0.record()
        out = bs.sample(x, h)
    e1.record()
    bs.check()
    if calls > 2:
        print(f"{workload}: {rows} rows, {e0.elapsed_time(e1) / (calls - 2) * 1e3:.1f} us per call")
    print(out[:4].cpu().numpy())
    bs.close()


if __name__ == "__main__":
    main()
