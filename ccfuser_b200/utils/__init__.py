from .dist import (env_rank, init_distributed, make_ep_dp_groups, get_torch_default_comm,
                   get_rank_0_in_comm, max_over_ranks, group_rank, group_size)
