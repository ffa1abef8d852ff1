"""Who is still there, decided on the host between steps.

Upstream's multi-GPU program has no failure handling: its replicas run under one tbb::parallel_for in one process
(apps/host-multi/main.cpp:157-181) and an exception in any of them ends the program.  With one process per GPU a
rank can go away on its own, and the ranks that stay must learn of it BEFORE their next launch: a kernel or a
collective that waits for a peer which no longer exists can only run into its time limit.  So every rank posts the
number of the step it has finished on a board all ranks can read, and before it launches step n it checks that
every peer has finished step n-1 and has not said goodbye.  Leaving is only allowed between steps, with nothing in
flight (synchronise first).  The board is a directory of one small file per rank, replaced atomically; one node is
the scope of this library, so a directory is enough and needs no server.

    board = StepBoard(path, rank, world)
    for step in range(n):
        board.wait_for_peers(step)         # raises PeerLeft / PeerTimeout: do NOT launch, abort the communicator
        run_step()                         # kernels + collectives
        synchronize()
        board.post(step + 1)               # or board.leave(step + 1) when this was the rank's last step
    board.leave()

post(n) therefore means "finished step n-1 and ready to join step n".  A rank whose host side fails, or stalls, does so
before it posts, and its peers' wait_for_peers ends with PeerLeft or PeerTimeout instead of a launch.  What the board
cannot cover is a rank that dies after it has posted; there the next collective's own time limit is the back stop
(NCCL communicator time-out, the bounded waits of the peer-exchange kernels with their status word).
"""
from __future__ import annotations

import os
import time


class PeerLeft(RuntimeError):
    def __init__(self, rank: int, step: int):
        super().__init__(f"rank {rank} left after step {step}")
        self.rank, self.step = rank, step


class PeerTimeout(RuntimeError):
    def __init__(self, rank: int, seen: int, wanted: int, seconds: float):
        super().__init__(f"rank {rank} has not finished step {wanted} after {seconds:.1f} s (last seen: {seen})")
        self.rank, self.seen, self.wanted = rank, seen, wanted


class StepBoard:
    LEFT = "left"

    def __init__(self, path: str, rank: int, world: int, timeout_s: float = 30.0, poll_s: float = 0.002):
        if not (0 <= rank < world):
            raise ValueError("StepBoard: rank outside the world")
        self.path, self.rank, self.world = path, rank, world
        self.timeout_s, self.poll_s = timeout_s, poll_s
        self.gone: set[int] = set()
        os.makedirs(path, exist_ok=True)
        self._write(f"0 alive")

    def _file(self, rank: int) -> str:
        return os.path.join(self.path, f"rank_{rank}")

    def _write(self, text: str) -> None:
        tmp = self._file(self.rank) + f".tmp{os.getpid()}"
        with open(tmp, "w") as f:
            f.write(text)
        os.replace(tmp, self._file(self.rank))

    def read(self, rank: int) -> tuple[int, bool]:
        """(steps finished, still there) of a rank; (-1, True) while it has not posted anything yet."""
        try:
            with open(self._file(rank)) as f:
                step, state = f.read().split()
            return int(step), state != self.LEFT
        except (FileNotFoundError, ValueError):
            return -1, True

    def post(self, steps_finished: int) -> None:
        self._write(f"{steps_finished} alive")
        self._posted = steps_finished

    def leave(self, steps_finished: int | None = None) -> None:
        """Say goodbye; only between steps, with none of this rank's kernels or collectives in flight.  A rank that
        leaves after step n calls leave(n) INSTEAD of post(n): a post followed by a goodbye would let a peer read
        "finished n, alive" in between and launch step n+1 against a rank that is about to go."""
        if steps_finished is None:
            steps_finished = getattr(self, "_posted", 0)
        self._write(f"{steps_finished} {self.LEFT}")

    def wait_for_peers(self, steps_finished: int, timeout_s: float | None = None) -> None:
        """Return once every peer has finished `steps_finished` steps.  A peer that left raises PeerLeft at once; a
        peer that stays silent raises PeerTimeout after the limit.  Either way the caller must not launch."""
        limit = self.timeout_s if timeout_s is None else timeout_s
        t0 = time.monotonic()
        pending = [r for r in range(self.world) if r != self.rank]
        while pending:
            still = []
            for r in pending:
                step, alive = self.read(r)
                if not alive:
                    self.gone.add(r)
                    raise PeerLeft(r, step)
                if step < steps_finished:
                    still.append((r, step))
            pending = [r for r, _ in still]
            if not pending:
                return
            waited = time.monotonic() - t0
            if waited > limit:
                r, step = still[0]
                self.gone.add(r)
                raise PeerTimeout(r, step, steps_finished, waited)
            time.sleep(self.poll_s)

    def survivors(self) -> list[int]:
        return [r for r in range(self.world) if r not in self.gone]
