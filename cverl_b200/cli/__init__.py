"""Command-line tools (``python -m cverl_b200.cli.<name>``): model inspection, forward dumps, weight
manifests, golden replay, the synthetic rollout batch source, and multi-GPU smokes."""
