"""Counter-based uniform numbers for sampling, keyed by (seed, request index,
step index) so that a request's draws do not depend on batching, on
preemption, or on what else is running.  andre-fu/prism draws from torch's
global generator (engine/scheduler.py:271, engine/executor.py:427), which
cannot be replayed."""

_M64 = (1 << 64) - 1


def uniform(seed: int, request_index: int, step_index: int) -> float:
    """In [0, 1) with 24 random bits: three rounds of the splitmix64 finaliser."""
    z = (seed * 0x9E3779B97F4A7C15 + request_index * 0xBF58476D1CE4E5B9
         + step_index * 0x94D049BB133111EB + 0x2545F4914F6CDD1D) & _M64
    for _ in range(3):
        z = (z + 0x9E3779B97F4A7C15) & _M64
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
        z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)
