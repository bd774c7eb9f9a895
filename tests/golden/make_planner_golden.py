"""Writes tests/golden/planner_golden.json from the reference's OWN compiled
planner (oracle/_ref/libtc_ref.so, built from the reference checkout by
`make -C oracle ref`).  Run where the reference checkout is mounted:

    python tests/golden/make_planner_golden.py
"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import oracle  # noqa: E402
from tests.test_oracle_planner import _random_requests  # noqa: E402


def main():
    ref = oracle.ref()
    cases = []
    for kw in _random_requests(160, seed=2026):
        cases.append({"request": kw, "plan": ref.plan_context(oracle.make_request(**kw))})
    with open(os.path.join(HERE, "planner_golden.json"), "w") as f:
        json.dump(cases, f, indent=0, sort_keys=True)
    print(f"wrote {len(cases)} cases")


if __name__ == "__main__":
    main()
