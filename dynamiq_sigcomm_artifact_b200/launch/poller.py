"""Command-file poller: run the lines that appear in a text file, one after another.

    python -m dynamiq_sigcomm_artifact_b200.launch.poller --command commands.txt [--global_seed 42]

The file is re-read every second; each new non-empty line is executed by the shell with
``GLOBAL_SEED=<seed>`` in its environment, ``cd <dir>`` changes the working directory of later
lines, and ``exit`` stops the poller.  This is how the reference queues simulation runs on a node
that is already reserved (simulations_llm/run_entry.py:1-53).
"""
from __future__ import annotations

import argparse
import os
import subprocess
import time
from typing import Callable, List, Optional


class CommandFilePoller:
    def __init__(self, path: str, global_seed: int = 42, poll_seconds: float = 1.0,
                 runner: Optional[Callable[[str, dict, str], int]] = None):
        self.path = os.path.abspath(path)
        self.seed = int(global_seed)
        self.poll_seconds = poll_seconds
        self.cwd = os.getcwd()
        self.done = 0  # lines consumed so far
        self.history: List[str] = []
        self.stopped = False
        self.runner = runner or self._shell

    @staticmethod
    def _shell(command: str, env: dict, cwd: str) -> int:
        return subprocess.run(command, shell=True, env=env, cwd=cwd).returncode

    def _pending(self) -> List[str]:
        try:
            with open(self.path) as f:
                lines = f.read().split("\n")
        except OSError:
            return []
        if lines and lines[-1] == "":
            lines.pop()  # a line counts once its newline has been written
        elif lines:
            lines.pop()  # the last line is still being written
        return lines[self.done:]

    def poll_once(self) -> bool:
        """Run every complete new line; returns False once ``exit`` was read."""
        if self.stopped:
            return False
        for line in self._pending():
            self.done += 1
            cmd = line.strip()
            if not cmd:
                continue
            if cmd == "exit":
                self.stopped = True
                return False
            if cmd == "cd" or cmd.startswith("cd "):
                target = cmd[3:].strip() or os.path.expanduser("~")
                self.cwd = target if os.path.isabs(target) else os.path.normpath(os.path.join(self.cwd, target))
                continue
            env = dict(os.environ, GLOBAL_SEED=str(self.seed))
            try:
                rc = self.runner(cmd, env, self.cwd)
            except Exception as e:  # a failing command must not stop the queue
                print(f"[poller] {cmd!r} failed: {type(e).__name__}: {e}", flush=True)
                rc = -1
            self.history.append(cmd)
            if rc:
                print(f"[poller] {cmd!r} exited with {rc}", flush=True)
        return True

    def run(self, max_polls: Optional[int] = None) -> int:
        polls = 0
        while self.poll_once():
            polls += 1
            if max_polls is not None and polls >= max_polls:
                break
            time.sleep(self.poll_seconds)
        return len(self.history)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--command", required=True, help="text file that receives one shell command per line")
    ap.add_argument("--global_seed", type=int, default=42)
    ap.add_argument("--poll_seconds", type=float, default=1.0)
    args = ap.parse_args(argv)
    CommandFilePoller(args.command, args.global_seed, args.poll_seconds).run()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
