"""rollout subpackage."""
