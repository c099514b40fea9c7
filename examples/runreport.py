"""Summarise a run directory: reward trajectory, throughput, memory, anomalies.

    python examples/runreport.py runs/<run-id>

Reads ``metrics.jsonl`` (and ``candidates.jsonl`` when present) the way ``ferrl report`` does.
Counterpart of ``crates/ferrl/examples/runreport.rs``.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ferrl_b200 import telemetry as T  # noqa: E402


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 1:
        print(__doc__)
        return 2
    run = T.RunDir.open(argv[0])
    rows = T.read_metrics(run.metrics_path)
    s = T.summarize(rows)
    print(f"run {run.run_id}: {s.steps} steps, reward {s.reward_first:.3f} -> {s.reward_last:.3f} (best {s.reward_best:.3f})")
    print(f"mean step {s.mean_step_secs:.3f} s, {s.mean_tokens_per_sec:.0f} tokens/s, final grad norm {s.final_grad_norm:.4f}, "
          f"peak device memory {s.peak_mem_bytes / 2 ** 30:.2f} GiB")
    for a in s.anomalies:
        print("anomaly:", a.kind, a.detail)
    return 0


if __name__ == "__main__":
    sys.exit(main())
