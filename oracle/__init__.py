"""Parity checker (test infrastructure only).

`oracle.port`      - plain-C restatement of the reference's fused-execution path.
`oracle.reference` - the reference's own headers compiled for the host (oracle/_ref).

Only tests, the smoke check and the benchmark's CPU-baseline legs may import this package.
"""
