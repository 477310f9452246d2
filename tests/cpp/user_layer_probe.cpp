// A layer written against the reference's plugin header (the shape of examples/sigmoid.h: clone,
// getName, a CPU forward(), dz and dz_star Jacobian entries) must still COMPILE against the host
// facade, and CNet::add must refuse it with a message, because the generic Jacobian loop that would
// call dz / dz_star (impl/cfunc.h:290-325) has no device form.  A layer that says it launches its own
// kernels is accepted.  No GPU is touched.
#include <cstdio>
#include <cstring>

#include "../../cnet_b200/host/cnet.h"

using namespace cnet_b200;

class JacobianOnly : public CFunc {
public:
	JacobianOnly(Uid uid, InSize n) : CFunc(uid, n, OutSize(n.value())) {}
	CFunc* clone(Uid uid) override { return new JacobianOnly(uid, InSize(in_size_)); }
	std::string getName() override { return "JacobianOnly_" + std::to_string(uid_); }
	void forward() override {}
	std::complex<float> dz(int out_indx, int in_indx) override { return out_indx == in_indx ? 1.f : 0.f; }
	std::complex<float> dz_star(int, int) override { return 0.f; }
};

class OwnKernels : public JacobianOnly {
public:
	OwnKernels(Uid uid, InSize n) : JacobianOnly(uid, n) {}
	bool runsOnDevice() const override { return true; }
};

int main() {
	CNet net;
	int x = net.add(new CInput(Uid(1), OutSize(8)));
	if (x != 1) { std::printf("FAIL input uid %d\n", x); return 1; }
	JacobianOnly* j = new JacobianOnly(Uid(2), InSize(8));
	int rc = net.add(j, {1});
	if (rc >= 0 || net.ok() || net.error().find("dz_star") == std::string::npos) {
		std::printf("FAIL a Jacobian-only layer was not refused: rc %d, '%s'\n", rc, net.error().c_str());
		return 1;
	}
	delete j;                                   // a refused layer stays the caller's
	net.clearError();
	rc = net.add(new OwnKernels(Uid(3), InSize(8)), {1});
	if (rc != 3 || !net.ok()) { std::printf("FAIL a device layer was refused: %s\n", net.error().c_str()); return 1; }
	CGelu g(Uid(9), InSize(4));                 // built-in layers: documented "not used" value
	if (g.dz(0, 0) == g.dz(0, 0)) { std::printf("FAIL built-in dz should be NaN\n"); return 1; }
	std::printf("OK\n");
	return 0;
}
