"""Drop-in MoE block and expert-store modules (same classes and signatures as bitsmoe.models)."""
