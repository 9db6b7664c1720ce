"""Small, self-terminating cases of the generated-operand kernels for profilers and for the per-role counters.

    python -m randumb_b200.profile_case                 # 2 launches each of the y-shaped and g-shaped product (for ncu -k regex:noise_)
    python -m randumb_b200.profile_case --staged        # 2 launches each of the noise fill and the two plain products on the staged S
                                                        # (for ncu -k "regex:dense_|noise_bf16")
    python -m randumb_b200.profile_case --roles         # per-role cycle counters of every kernel variant at the headline shapes
    python -m randumb_b200.profile_case --tokens 2048 --out 16384 --dc 1024

The default sizes keep the device footprint around 150 MB and each launch near 0.1-0.3 ms, so a capture with
many replay passes ends by itself; the inputs still exceed the 126 MB L2 on the g-shaped product.
"""
from __future__ import annotations

import argparse

import torch

from . import _lib
from . import kernels as K

ROLE_NAMES = ["mma_wait_full_or_A", "mma_wait_B", "mma_wait_tmem", "mma_total", "tma_wait_free", "gen_wait_free", "gen_busy",
              "epilogue_busy"]


def run_small(tokens: int, out: int, dc: int, seed: int = 42) -> None:
    z = torch.randn(tokens, dc, device="cuda").bfloat16()
    dy = torch.randn(tokens, out, device="cuda").bfloat16()
    for _ in range(2):
        K.gemm_noise(z, out, seed, False, impl=K.IMPL_UMMA)       # y = z S^T
        K.gemm_noise(dy, dc, seed, True, impl=K.IMPL_UMMA)        # g = dY S
    torch.cuda.synchronize()
    K.check_status()


def run_staged(tokens: int, out: int, dc: int, seed: int = 42) -> None:
    """The path the linear entry points take for 1024 tokens or more: S hashed once into bf16, then the plain products."""
    z = torch.randn(tokens, dc, device="cuda").bfloat16()
    dy = torch.randn(tokens, out, device="cuda").bfloat16()
    assert K.linear_stages_noise(tokens, 8, out, dc, torch.bfloat16, K.PATH_FACTORED)
    for _ in range(2):
        K.noise_product(z, out, seed, False)       # noise fill + y = z S^T
        K.noise_product(dy, dc, seed, True)        # noise fill + g = dY S
    torch.cuda.synchronize()
    K.check_status()


def run_roles(tokens: int, out: int, dc: int, seed: int = 42) -> None:
    L = _lib.lib()
    z = torch.randn(tokens, dc, device="cuda").bfloat16()
    dy = torch.randn(tokens, out, device="cuda").bfloat16()
    prof = torch.zeros(148 * 16, dtype=torch.int64, device="cuda")
    for tile in (1, 3, 7, 8):
        prev = K.set_option(_lib.OPT_NOISE_TILE, tile)
        try:
            for which, fn in (("y", lambda: K.gemm_noise(z, out, seed, False, impl=K.IMPL_UMMA)),
                              ("g", lambda: K.gemm_noise(dy, dc, seed, True, impl=K.IMPL_UMMA))):
                for _ in range(3):
                    fn()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(5):
                    fn()
                e1.record()
                torch.cuda.synchronize()
                prof.zero_()
                L.rdb_set_profile_buffer(prof.data_ptr(), prof.numel() * 8)
                fn()
                torch.cuda.synchronize()
                L.rdb_set_profile_buffer(None, 0)
                p = prof.view(148, 16).double()[:, :8]
                issuing = p[p[:, 3] > 0]
                total = float(issuing[:, 3].mean())
                gens = p[p[:, 6] > 0]
                vals = issuing.mean(0)
                vals[4:7] = gens.mean(0)[4:7]
                print(f"variant {tile} {which}: {e0.elapsed_time(e1) / 5:.4f} ms  mma_total {total / 1e3:.0f} kcycles  " +
                      "  ".join(f"{n}={100 * float(v) / total:.0f}%" for n, v in zip(ROLE_NAMES, vals.tolist())))
        finally:
            K.set_option(_lib.OPT_NOISE_TILE, prev)
    K.check_status()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--roles", action="store_true")
    ap.add_argument("--staged", action="store_true")
    ap.add_argument("--tokens", type=int, default=None)
    ap.add_argument("--out", type=int, default=16384)
    ap.add_argument("--dc", type=int, default=1024)
    a = ap.parse_args()
    if a.roles:
        run_roles(a.tokens or 8192, a.out, a.dc)
    elif a.staged:
        run_staged(a.tokens or 4096, a.out, a.dc)
    else:
        run_small(a.tokens or 2048, a.out, a.dc)
    print("ok")


if __name__ == "__main__":
    main()
