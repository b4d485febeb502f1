"""Host-side fault injection for the failure-detection and restart tests.

A fault is a thing a PROCESS does between two steps, on the host, with none of its kernels or
collectives in flight: raise an exception, exit with a code, or stop making progress (sleep).  Nothing
here makes a device fault, trap or spin; a rank on a GPU synchronises its device before it leaves.

The fault is described by one environment variable so that a launcher can plant it in a child:

    CVERL_B200_INJECT_FAULT="rank=1,step=2,kind=exit[,code=17][,attempt=0]"

``kind`` is ``raise`` (a ``RuntimeError`` that travels the trainer's normal error path and is published
to the peers' watchdogs), ``exit`` (``os._exit``: no clean-up, no message - a killed process) or
``stall`` (sleeps until it is terminated - a process that is alive but stuck).  ``attempt`` restricts
the fault to one attempt of a supervised job (``CVERL_LAUNCH_ATTEMPT``, set by
``cverl_b200.cli.launch``; default 0), so that the restarted job runs through.

The reference has no fault injection (its launcher only ``wait``s,
tools/distributed/run_qwen_pp_tp_ppo_trainer.sh:123-128).
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass
from typing import Optional

ENV = "CVERL_B200_INJECT_FAULT"
ATTEMPT_ENV = "CVERL_LAUNCH_ATTEMPT"
KINDS = ("raise", "exit", "stall")


class InjectedFault(RuntimeError):
    pass


@dataclass
class HostFault:
    rank: int
    step: int
    kind: str
    code: int = 17
    attempt: int = 0

    @staticmethod
    def parse(spec: str) -> "HostFault":
        fields = {}
        for part in spec.split(","):
            if not part.strip():
                continue
            if "=" not in part:
                raise ValueError(f"{ENV}: expected key=value, got {part!r}")
            k, v = part.split("=", 1)
            fields[k.strip()] = v.strip()
        unknown = set(fields) - {"rank", "step", "kind", "code", "attempt"}
        if unknown:
            raise ValueError(f"{ENV}: unknown keys {sorted(unknown)}")
        for need in ("rank", "step", "kind"):
            if need not in fields:
                raise ValueError(f"{ENV}: {need}= is required")
        if fields["kind"] not in KINDS:
            raise ValueError(f"{ENV}: kind must be one of {KINDS}")
        return HostFault(rank=int(fields["rank"]), step=int(fields["step"]), kind=fields["kind"],
                         code=int(fields.get("code", 17)), attempt=int(fields.get("attempt", 0)))

    @staticmethod
    def from_env(environ=None) -> Optional["HostFault"]:
        environ = os.environ if environ is None else environ
        spec = environ.get(ENV, "")
        return HostFault.parse(spec) if spec else None

    def due(self, rank: int, step: int, environ=None) -> bool:
        environ = os.environ if environ is None else environ
        return rank == self.rank and step == self.step and int(environ.get(ATTEMPT_ENV, "0") or 0) == self.attempt

    def fire(self, rank: int, step: int, *, sync=None, sleep=time.sleep, exit_fn=os._exit) -> None:
        """Call at the top of a step.  ``sync`` (e.g. ``torch.cuda.synchronize``) runs first so that the rank
        leaves with nothing in flight."""
        if not self.due(rank, step):
            return
        if sync is not None:
            sync()
        if self.kind == "raise":
            raise InjectedFault(f"injected fault on rank {rank} at step {step}")
        if self.kind == "exit":
            exit_fn(self.code)
            return
        while True:                         # "stall": alive, silent, until the supervisor ends the process
            sleep(0.25)
