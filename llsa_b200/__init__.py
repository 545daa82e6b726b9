"""llsa_b200: B200-native LLSA hot path."""
