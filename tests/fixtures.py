"""Recorded routing statistics used as skew fixtures.

RECORDED_COUNTS[r][e] = slots that rank r routed to expert e in one step of a 4-GPU, 64-expert, top-2 run with 4096
tokens per GPU: the values stored in the reference repository at mix_moe/mix_moe/all_expert_count.pt (a [4, 64] int64
tensor; every row sums to 8192). A handful of experts draw most of the load and the hot experts differ by rank, which
is what routing, capacity dropping and placement planning have to cope with in practice."""

RECORDED_COUNTS = [
    [82, 1, 0, 3, 291, 132, 268, 1, 0, 1238, 5, 0, 8, 53, 202, 5, 0, 5, 6, 43, 10, 73, 568, 0, 0, 0, 2, 30, 0, 1, 1, 1, 3, 0, 3885, 2, 85, 1, 0, 0, 10, 0, 0, 122, 0, 5, 0, 0, 0, 78, 904, 3, 0, 41, 0, 0, 0, 0, 0, 19, 0, 0, 0, 5],
    [82, 0, 3, 0, 0, 0, 0, 0, 0, 12, 8, 12, 88, 1, 0, 0, 5, 0, 5, 0, 8, 1, 0, 1, 31, 14, 16, 0, 0, 2, 0, 0, 1, 0, 308, 0, 0, 28, 12, 52, 0, 387, 0, 390, 0, 0, 823, 0, 94, 0, 11, 450, 44, 0, 0, 0, 0, 0, 3953, 1313, 0, 0, 0, 37],
    [0, 0, 1, 0, 0, 0, 276, 23, 0, 0, 10, 292, 29, 26, 0, 947, 0, 8, 0, 1, 61, 3, 1, 0, 66, 0, 14, 0, 0, 0, 1242, 0, 47, 0, 1446, 6, 309, 0, 0, 0, 2, 0, 0, 4, 217, 0, 2, 5, 62, 0, 0, 3, 0, 273, 2808, 4, 4, 0, 0, 0, 0, 0, 0, 0],
    [58, 57, 80, 0, 5, 4, 85, 0, 2, 0, 198, 33, 0, 0, 11, 1, 27, 227, 56, 1, 0, 17, 0, 1, 256, 0, 0, 702, 1, 3, 0, 0, 0, 234, 56, 3, 170, 179, 22, 0, 59, 40, 0, 287, 81, 32, 0, 0, 3218, 0, 0, 128, 42, 0, 10, 0, 23, 0, 0, 0, 263, 1520, 0, 0],
]
