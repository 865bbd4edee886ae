"""Summarise an .ncu-rep (raw page) into profiles/ (tracked evidence)."""
import csv
import io
import os
import re
import subprocess
import sys
from collections import Counter

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WANT = ["gpu__time_duration.sum", "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active",
        "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed", "sm__inst_executed_pipe_xu.avg.pct_of_peak_sustained_active",
        "sm__pipe_fmaheavy_cycles_active.avg.pct_of_peak_sustained_elapsed", "smsp__issue_active.avg.pct_of_peak_sustained_active",
        "sm__throughput.avg.pct_of_peak_sustained_elapsed", "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed",
        "dram__bytes_read.sum", "dram__bytes_write.sum", "launch__registers_per_thread", "launch__grid_size",
        "launch__block_size", "launch__shared_mem_per_block_dynamic", "sm__warps_active.avg.pct_of_peak_sustained_active",
        "l1tex__data_bank_conflicts_pipe_lsu_mem_shared.sum", "sm__cycles_elapsed.avg.per_second"]


def ncu_summary(rep, out_md, title):
    raw = subprocess.run(["ncu", "-i", rep, "--page", "raw", "--csv"], capture_output=True, text=True).stdout
    rows = list(csv.reader(io.StringIO(raw)))
    hdr, units = rows[0], rows[1]
    lines = [f"# {title}", "", f"source: `{os.path.basename(rep)}` (ncu --set full --clock-control none), B200", ""]
    seen = Counter()
    for r in rows[2:]:
        name = r[hdr.index("Kernel Name")]
        short = re.sub(r"\(.*", "", name)
        seen[short] += 1
        if seen[short] > 1:
            continue
        lines.append(f"## {short}")
        lines.append("")
        lines.append("| metric | value | unit |")
        lines.append("|---|---|---|")
        for w in WANT:
            if w in hdr:
                i = hdr.index(w)
                lines.append(f"| {w} | {r[i]} | {units[i]} |")
        lines.append("")
    open(out_md, "w").write("\n".join(lines) + "\n")


if __name__ == "__main__":
    os.makedirs(os.path.join(ROOT, "profiles"), exist_ok=True)
    if len(sys.argv) > 1:
        ncu_summary(sys.argv[1], os.path.join(ROOT, "profiles", sys.argv[2]), sys.argv[3] if len(sys.argv) > 3 else "ncu summary")
