// Fixture generator: real positions from a binpack file through the reference project's own
// feature extractors (HalfKAv2_hm, Full_Threats, PP_3Wide).  Built and run by
// tests/golden/make_golden.py against a reference checkout:
//
//     g++ -std=c++20 -O1 -I<checkout>/data_loader/cpp dump_features.cpp -o dump_features -lpthread
//     ./dump_features <file.binpack> <count> <stride>
//
// It includes the reference's training_data_loader.cpp where it lies (nothing is copied) and
// prints one line per position: the 64 board squares as piece codes (0 = empty, else
// 1 + 2 * (type - 1) + is_black for pawn..king = types 1..6), the side to move (0 = white),
// then for each perspective (white, black) and each extractor the list length and the indices.
#include "training_data_loader.cpp"

#include <cstdio>
#include <cstdlib>

int main(int argc, char** argv) {
    if (argc < 4) {
        std::fprintf(stderr, "usage: dump_features file.binpack count stride\n");
        return 2;
    }
    const int count = std::atoi(argv[2]), stride = std::atoi(argv[3]);
    binpack::CompressedTrainingDataEntryReader reader(argv[1]);
    int seen = 0, written = 0;
    int feats[512];
    while (reader.hasNext() && written < count) {
        const auto e = reader.next();
        if (seen++ % stride != 0) continue;
        const auto& pos = e.pos;
        for (int sq = 0; sq < 64; ++sq) {
            const Piece p = pos.pieceAt(Square(sq));
            int code = 0;
            if (p != Piece::none()) code = 1 + 2 * static_cast<int>(p.type()) + (p.color() == Color::Black ? 1 : 0);
            std::printf("%d ", code);
        }
        std::printf("%d", pos.sideToMove() == Color::White ? 0 : 1);
        for (Color c : {Color::White, Color::Black}) {
            auto dump = [&](std::pair<int, int> r) {
                std::printf(" %d", r.first);
                for (int i = 0; i < r.first; ++i) std::printf(" %d", feats[i]);
            };
            dump(HalfKAv2_hm::fill_features_sparse(e, feats, c));
            dump(FullThreats::fill_features_sparse(e, feats, c));
            dump(PP_3Wide::fill_features_sparse(e, feats, c));
        }
        std::printf("\n");
        ++written;
    }
    return written > 0 ? 0 : 1;
}
