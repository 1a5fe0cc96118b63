from bitsmoe_b200.models.base_mlp import BitsMoE_BaseMoeMLP


class BitsMoE_Qwen3MoeMLP(BitsMoE_BaseMoeMLP):
    """Packed expert container of the Qwen3Moe family (bitsmoe/models/qwen3moe/bitsmoe_mlp.py)."""
