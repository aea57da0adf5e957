"""minfer — B200-native attention path behind the reference's op surface."""
