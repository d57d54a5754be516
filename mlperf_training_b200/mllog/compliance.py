"""``python -m mlperf_training_b200.mllog.compliance <trial.log>``: structural MLLOG check of one
trial log; exit status 0 when compliant."""
from __future__ import annotations

import sys
from pathlib import Path

from .core import check_compliance, parse_log


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) == 1 and argv[0] in ("-h", "--help"):
        print("usage: compliance <logfile>   (checks the :::MLLOG lines of one trial log; exit 0 = compliant)")
        return 0
    if len(argv) != 1:
        print("usage: compliance <logfile>", file=sys.stderr)
        return 2
    records = parse_log(Path(argv[0]).read_text(errors="replace"))
    problems = check_compliance(records)
    if not records:
        problems.append("no :::MLLOG lines")
    for p in problems:
        print(f"COMPLIANCE: {p}")
    print(f"compliance: {'SUCCESS' if not problems else 'FAILED'} ({len(records)} events)")
    return 0 if not problems else 1


if __name__ == "__main__":
    sys.exit(main())
