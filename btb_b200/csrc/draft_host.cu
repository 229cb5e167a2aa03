// Host side of speculative decoding, native: the n-gram proposer's index, the merge of its continuations into one tree
// of guesses, and the walk that accepts a branch. No device code in this file.
//
// What it must reproduce is btb's drafting (btb/draft.py:8-113 `NGramProposer`, btb/engine/generate.py:94-117
// `_chains_tree`, :765-795 the accept walk): for every order n in [n_min, n_max] each n-gram of the text remembers who
// followed it - how often and where last; the continuations of the text's tail are proposed longest order first and,
// within an order, most frequent (then most recent) follower first, a continuation that is a prefix of an earlier one
// dropped; the continuations are merged by shared prefix into a tree of at most `budget` guesses whose nodes are
// numbered parents first. The proposals and the tree are the reference's to the element (checked against fixtures made
// by the reference's own functions); the index underneath is this file's: one open-addressed table an order, keyed by a
// hash of the n-gram and verified against the text itself, so nothing is allocated per n-gram but a small follower list.
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <new>
#include <vector>

#include "btb_b200_internal.h"

namespace {

struct Follower {
    int tok, count, at;  // `at`: the follower's position in the text at its latest occurrence
};
struct Gram {
    int first = -1;  // where the n-gram first stood in the text (the key is read back from there); -1: empty slot
    std::vector<Follower> next;
};
struct OrderIndex {
    int n = 0;
    std::vector<Gram> slots;  // open addressing, a power of two
    size_t used = 0;
};
struct Proposer {
    int n_max, n_min, followers;
    std::vector<int> text;
    std::vector<OrderIndex> orders;  // orders[n - n_min]
};

uint64_t gram_hash(const int* p, int n) {
    uint64_t h = 0x9E3779B97F4A7C15ull ^ (uint64_t)n;
    for (int i = 0; i < n; ++i) {
        h ^= (uint64_t)(uint32_t)p[i] + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
        h *= 0xFF51AFD7ED558CCDull;
        h ^= h >> 33;
    }
    return h;
}

Gram* find_slot(OrderIndex& ix, const std::vector<int>& text, const int* key, bool insert, int first_at) {
    if (ix.slots.empty()) {
        if (!insert) return nullptr;
        ix.slots.resize(64);
    }
    if (insert && (ix.used + 1) * 4 > ix.slots.size() * 3) {  // grow at three quarters full
        std::vector<Gram> old;
        old.swap(ix.slots);
        ix.slots.resize(old.size() * 2);
        ix.used = 0;
        for (Gram& g : old) {
            if (g.first < 0) continue;
            size_t i = gram_hash(text.data() + g.first, ix.n) & (ix.slots.size() - 1);
            while (ix.slots[i].first >= 0) i = (i + 1) & (ix.slots.size() - 1);
            ix.slots[i] = std::move(g);
            ++ix.used;
        }
    }
    size_t i = gram_hash(key, ix.n) & (ix.slots.size() - 1);
    for (;;) {
        Gram& g = ix.slots[i];
        if (g.first < 0) {
            if (!insert) return nullptr;
            g.first = first_at;
            ++ix.used;
            return &g;
        }
        if (memcmp(text.data() + g.first, key, sizeof(int) * ix.n) == 0) return &g;
        i = (i + 1) & (ix.slots.size() - 1);
    }
}

void extend_one(Proposer& P, int tok) {
    P.text.push_back(tok);
    const int len = (int)P.text.size();
    for (OrderIndex& ix : P.orders) {
        const int start = len - ix.n - 1;  // the n-gram that this token follows
        if (start < 0) continue;
        Gram* g = find_slot(ix, P.text, P.text.data() + start, true, start);
        bool seen = false;
        for (Follower& f : g->next)
            if (f.tok == tok) {
                ++f.count;
                f.at = start + ix.n;
                seen = true;
                break;
            }
        if (!seen) g->next.push_back(Follower{tok, 1, start + ix.n});
    }
}

// the tail's continuations of up to v tokens, flattened: chain c is toks[offs[c] .. offs[c + 1]), found by order[c]
void propose(Proposer& P, int v, std::vector<int>& toks, std::vector<int>& offs, std::vector<int>& order) {
    toks.clear(), order.clear();
    offs.assign(1, 0);
    if (v <= 0) return;
    const int len = (int)P.text.size();
    for (int n = P.n_max; n >= P.n_min; --n) {
        if (len < n) continue;
        OrderIndex& ix = P.orders[n - P.n_min];
        Gram* g = find_slot(ix, P.text, P.text.data() + len - n, false, -1);
        if (g == nullptr) continue;
        std::vector<Follower> best(g->next);
        std::sort(best.begin(), best.end(), [](const Follower& a, const Follower& b) {
            return a.count != b.count ? a.count > b.count : a.at > b.at;  // positions are distinct: a total order
        });
        if ((int)best.size() > P.followers) best.resize(P.followers);
        for (const Follower& f : best) {
            const int m = std::min(v, len - f.at);
            if (m <= 0) continue;
            const int* c = P.text.data() + f.at;
            bool covered = false;
            for (size_t k = 0; k + 1 < offs.size() && !covered; ++k) {
                const int l = offs[k + 1] - offs[k];
                covered = l >= m && memcmp(toks.data() + offs[k], c, sizeof(int) * m) == 0;
            }
            if (covered) continue;
            toks.insert(toks.end(), c, c + m);
            offs.push_back((int)toks.size());
            order.push_back(n);
        }
    }
}

// chains merged by shared prefix. Node 0 is the root; node j > 0 carries guesses[j - 1]. A chain that meets the budget
// stops there; later chains may still descend through nodes that exist.
int merge(const int* toks, const int* offs, int n_chains, int budget, int* guesses, int* parents, int* depth) {
    int n_guesses = 0;
    parents[0] = -1, depth[0] = 0;
    for (int c = 0; c < n_chains; ++c) {
        int node = 0;
        for (int d = 0; d < offs[c + 1] - offs[c]; ++d) {
            const int t = toks[offs[c] + d];
            int child = -1;
            for (int j = 1; j <= n_guesses && child < 0; ++j)
                if (parents[j] == node && guesses[j - 1] == t) child = j;
            if (child < 0) {
                if (n_guesses >= budget) break;
                child = ++n_guesses;
                guesses[child - 1] = t, parents[child] = node, depth[child] = d + 1;
            }
            node = child;
        }
    }
    return n_guesses;
}

}  // namespace

extern "C" void* btb_b200_ngram_new(int n_max, int n_min, int followers) {
    if (n_min < 1 || n_max < n_min || n_max > 64) return nullptr;
    Proposer* P = new (std::nothrow) Proposer();
    if (P == nullptr) return nullptr;
    P->n_max = n_max, P->n_min = n_min, P->followers = followers < 1 ? 1 : followers;
    P->orders.resize(n_max - n_min + 1);
    for (int n = n_min; n <= n_max; ++n) P->orders[n - n_min].n = n;
    return P;
}

extern "C" void btb_b200_ngram_free(void* h) { delete static_cast<Proposer*>(h); }

extern "C" int btb_b200_ngram_extend(void* h, const long long* toks, int n) {
    if (!h || (n > 0 && !toks)) return B2_ERR_NULL;
    if (n < 0) return B2_ERR_DOMAIN;
    Proposer& P = *static_cast<Proposer*>(h);
    for (int i = 0; i < n; ++i) extend_one(P, (int)toks[i]);
    return B2_OK;
}

extern "C" int btb_b200_ngram_length(void* h) { return h ? (int)static_cast<Proposer*>(h)->text.size() : B2_ERR_NULL; }

/* the tail's continuations: chain c is toks[offs[c] .. offs[c + 1]) found by an n-gram of order[c]; at most max_chains
 * chains of at most v tokens (toks holds max_chains * v, offs max_chains + 1, order max_chains) */
extern "C" int btb_b200_ngram_chains(void* h, int v, int max_chains, int* toks, int* offs, int* order, int* n_chains) {
    if (!h || !toks || !offs || !order || !n_chains) return B2_ERR_NULL;
    if (max_chains < 0) return B2_ERR_DOMAIN;
    std::vector<int> t, o, ord;
    propose(*static_cast<Proposer*>(h), v, t, o, ord);
    const int n = std::min((int)ord.size(), max_chains);
    for (int c = 0; c <= n; ++c) offs[c] = o[c];
    if (n > 0) memcpy(toks, t.data(), sizeof(int) * o[n]);
    if (n > 0) memcpy(order, ord.data(), sizeof(int) * n);
    *n_chains = n;
    return B2_OK;
}

extern "C" int btb_b200_chains_tree(const int* toks, const int* offs, int n_chains, int budget, int* guesses, int* parents,
                                    int* depth, int* n_guesses) {
    if (!offs || !guesses || !parents || !depth || !n_guesses || (n_chains > 0 && !toks)) return B2_ERR_NULL;
    if (n_chains < 0 || budget < 0) return B2_ERR_DOMAIN;
    *n_guesses = merge(toks, offs, n_chains, budget, guesses, parents, depth);
    return B2_OK;
}

/* the tail's continuations merged straight into a tree: btb_b200_ngram_chains then btb_b200_chains_tree */
extern "C" int btb_b200_ngram_tree(void* h, int v, int budget, int* guesses, int* parents, int* depth, int* n_guesses) {
    if (!h || !guesses || !parents || !depth || !n_guesses) return B2_ERR_NULL;
    if (budget < 0) return B2_ERR_DOMAIN;
    std::vector<int> t, o, ord;
    propose(*static_cast<Proposer*>(h), v, t, o, ord);
    *n_guesses = merge(t.data(), o.data(), (int)ord.size(), budget, guesses, parents, depth);
    return B2_OK;
}

/* the accepted branch: from the root, the child whose guess is its parent's own pick, while there is one. picks [n_nodes]
 * (node j's pick), guesses [n_nodes - 1], parents [n_nodes]; path receives at most n_nodes node numbers, the root first */
extern "C" int btb_b200_tree_walk(const long long* picks, const int* guesses, const int* parents, int n_nodes, int* path,
                                  int* n_path) {
    if (!picks || !parents || !path || !n_path || (n_nodes > 1 && !guesses)) return B2_ERR_NULL;
    if (n_nodes < 1) return B2_ERR_DOMAIN;
    int node = 0, n = 0;
    path[n++] = 0;
    for (;;) {
        int child = -1;
        for (int j = node + 1; j < n_nodes && child < 0; ++j)  // children are numbered after their parent
            if (parents[j] == node && (long long)guesses[j - 1] == picks[node]) child = j;
        if (child < 0) break;
        path[n++] = node = child;
    }
    *n_path = n;
    return B2_OK;
}
