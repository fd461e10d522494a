"""Run by tests/test_gpu_switches.py in a process of its own (the IERT_* switches are read from
the environment when the libraries load): a fixed workload through the engine and the
projection kernel, its results saved with torch.save to the path given as the only argument.

  * Tiny A in bfloat16: four prompts of unequal lengths in one step, then eight tokens each;
  * two layers at 7B sizes in bfloat16: a 300-token prompt whole, then three requests batched,
    their last 32 / 5 / 17 tokens one by one (split-K projections, decode attention over
    several pages, a window of 160 that cuts the longest request);
  * the projection kernel alone where the order of its tiles and the cut of its last wave
    matter: 2,400 x 14,336 activations (above 64 MB) and 2,048 tokens against 4,096 x 14,336.
"""
import os
import sys

import torch

TESTS = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(TESTS))
sys.path.insert(0, TESTS)

from helpers import TINY_A, prompts_for                                 # noqa: E402
from test_gpu_full_size import CFG, LENGTHS, run_batched_with_tails     # noqa: E402


def main(path: str) -> None:
    from inference_engine_rust_b200 import LoadedModel
    from inference_engine_rust_b200.csrc import bindings as B
    out = {}
    tiny = LoadedModel.random(dict(TINY_A), seed=3, dtype="bfloat16", std=0.1)
    eng = tiny.session(max_tokens=64 * 8, poison_cache=True).engine
    prompts = prompts_for(TINY_A, [5, 11, 23, 70], seed=2)
    slots = [eng.open_sequence() for _ in prompts]
    rows = [eng.step(list(zip(slots, prompts)), want="all").clone()]
    g = torch.Generator().manual_seed(1)
    for _ in range(8):
        toks = torch.randint(0, TINY_A["vocab_size"], (len(slots),), generator=g).tolist()
        rows.append(eng.step([(s, [t]) for s, t in zip(slots, toks)], want="last").clone())
    eng.check_device()
    out["tiny"] = torch.cat(rows).cpu()

    big = LoadedModel.random(CFG, seed=5, dtype="bfloat16", std=0.02, on_device=True)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, CFG["vocab_size"], (n,), generator=g).tolist() for n in LENGTHS]
    eng = big.session(max_tokens=64 * 12, poison_cache=True).engine
    s = eng.open_sequence()
    out["whole"] = eng.step([(s, prompts[0])], want="all").cpu()
    eng.close_sequence(s)
    eng.check_device()
    out["cut"] = torch.cat(run_batched_with_tails(big, prompts, tails=[32, 5, 17])).cpu()

    err = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    for M, N, K in ((2400, 256, 14336), (2048, 4096, 14336)):
        g = torch.Generator(device="cuda:0").manual_seed(M + N + K)
        x = torch.randn(M, K, device="cuda:0", generator=g).bfloat16()
        w = (torch.randn(N, K, device="cuda:0", generator=g) * 0.5).bfloat16()
        res = torch.randn(M, N, device="cuda:0", generator=g)
        want = (x.double() @ w.double().t() + res.double())
        assert B.gemm_tc(x, w, res, M, B.GEMM_ADD_RESIDUAL, err, B.stream_ptr())
        torch.cuda.synchronize()
        out[f"gemm_{M}x{N}x{K}"] = res.cpu()
        out[f"gemm_{M}x{N}x{K}_err"] = float((res.double() - want).abs().max())
    assert err.item() == 0, B.describe_error_bits(err.item())
    torch.save(out, path)


if __name__ == "__main__":
    main(sys.argv[1])
