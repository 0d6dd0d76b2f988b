"""Fixed constants of the layer (values shared with the reference's python/zepp/constants.py so
capacities and swap lists come out identical)."""
SWAP_MAX_MOVES = 8               # changed slots per rank one swap decision may produce
CAPACITY_CUSHION_PER_RANK = 8    # rows added per rank on top of the provable bounds
RELAY_SLOTS = 2                  # multiplier of the per-round relay demand (inter-node term of the demands)
SHARE_BITS = 20                  # fixed-point scale of a replica's load share in the placement
WAIT_LIMIT_MS = 4000             # bound of every device-side wait
