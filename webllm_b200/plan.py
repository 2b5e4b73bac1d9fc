"""The reference's split-K planner, kept for hosts that rebuild its launch list.

``plan_gemv_split`` restates ``planGemvSplit`` (src/model/qwen.ts:42-74) exactly. It is a heuristic
tuned for the reference's integrated GPU (256 workgroups to saturate it); the CUDA library plans for 148
SMs instead and reports its own choice through ``Gpu.plan`` (``wb_plan_query``).
"""
GEMV_SPLIT_TARGET_WG = 256
GEMV_SPLIT_MAX = 64


def plan_gemv_split(wg_n: int, K: int) -> int:
    if wg_n >= GEMV_SPLIT_TARGET_WG:
        return 1
    s = 1
    for cand in (8, 16, 32, GEMV_SPLIT_MAX):
        if K % cand == 0 and (K // cand) % 2 == 0:
            s = cand
            if wg_n * cand >= GEMV_SPLIT_TARGET_WG:
                break
    return s
