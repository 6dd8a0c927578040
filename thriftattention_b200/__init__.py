"""B200-native (sm_100a) selective mixed-precision attention."""
