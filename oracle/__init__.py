"""TEST INFRASTRUCTURE ONLY: CPU restatement of WebDNN's cpu backend (see cpu_ops.c header).

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this package.
"""
