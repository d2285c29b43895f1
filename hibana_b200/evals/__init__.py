"""Quality and speed tooling that runs against this engine: the lossy-change gate, head-to-head speed runs and
task evaluation. Reference: tools/lossy_gate.py, tools/h2h_pr.py, tools/evaluate.py."""
