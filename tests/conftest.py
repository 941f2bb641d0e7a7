import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests"), os.path.join(ROOT, "tests", "golden")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_terminal_summary(terminalreporter):
    """Measured ratios of the fp64-arbitrated comparisons (helpers.assert_arbitrated): error against the fp64 run over
    the fp32 noise of the reference restatement, worst element per call site."""
    import helpers
    if not helpers.ARBITER_RATIOS:
        return
    terminalreporter.write_line("fp64-arbitrated comparisons: max|got - ref64| / max|ref32 - ref64| (bar: 4)")
    groups = {}
    for what, r in helpers.ARBITER_RATIOS.items():
        key = what.rsplit(" ", 1)[0]
        groups[key] = max(groups.get(key, 0.0), r)
    for key in sorted(groups):
        r = groups[key]
        terminalreporter.write_line("  %-60s %s" % (key, "%.2f" % r if r != float("inf") else
                                                    "fp32 and fp64 runs of the reference coincide; error within the bar"))
