"""Grid constants of the GGUF i-quant block formats (IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S, IQ1_S, IQ1_M).

These tables are part of the file format: an index stored in a block selects eight (IQ2, IQ1) or four (IQ3) magnitudes.
They are kept as zlib-compressed little-endian arrays in base85; ``grid(name)`` unpacks one on first use into a uint8
array [entries, values-per-entry] (IQ1: int8 in {-1, 0, 1}). ``KSIGNS`` maps a 7-bit sign index to the 8-bit sign mask
(the eighth bit is the parity of the other seven)."""
import base64
import zlib

import numpy as np

_PACKED = {
    "IQ2XXS_GRID": ("uint64", 256,
        "c-n<kTax4;4EyB@I)m<izZopam@Ku^)hQBU{E%d4E&b>fxHsq(3r_=n4Cxii2fhcX6~8yy=H-xCnP)kKudid^6CjRxJ3be4Uyd=I"
        "j{w*fwZ|(U6PT%t@DbVv?Z?mLOpr;GNtoJ4m9ot-k-`QDN`o)tejn*Lv*5(&E5S(@p%SYKIy*X>36x`(0gsC^8_;}#jPvu7Phf$+"
        "02af7WdcrFAV9wXmU|mL0Oy8z0G=z6I`xH%fQmGT5JzQP%B#qOknWbK9FYt$rBAPt%_L-M_eiXvJVaHog6j~66{xATlr{-<N9>m("
        "b}Oop{fB5{5%F~Fb#(!(=784>9f9B@6z3ZGn+3q@y5w7NMpY%0OHh0Z3zQ<Fp}HFai&FZ;r^6-6(dkM+dDHD`JHdFt**(`9zu`Fo"
        "W`wM6iK>gf<6bzzq4!#b0$*AH=425hj$4AKAuntsz5g`=c{PM$QGaO~vq6ANtO33ng?jEuHa|Q0oOA+FY%`KxT;0`cj>=}tlF^Wz"
        "8ss$rdn_0Q&s{ou`ooeoW=4@_)T1%oYtg!=rlGBUddA1N7%=TppnyWya#s6Pe|25{Va|Z|)S)EkDqE31?*x|A"
    ),
    "IQ2XS_GRID": ("uint64", 512,
        "c-nPW(Us&d2>W#lszLqtHxrOBIPvbwahpkO5R&k$l|NJj<_#)hVLU)ZaK1oAU@m~A1+)+q|BsD@sR+!Cu=u$l75`6-1h6m?`M)+2"
        "f-WaU#pkJ>C>5V{dg4^X;%6aLd|vB?Vd1+#QlG2POToULhdTgR_yht=KpcQP+jl_z|Bwxn)syie4KON36%D}H{R2oU28<0@EDV5o"
        "0PU@AKpP8R1|AEa4RFe5Bak~+LtN6?kcURSF?53vl&D6zH_piy6%ESS$mj|;l&{9}WICDaW;FD-#;b%CWei1d5aGWKbw478icy$="
        "lQ3=;FbRag#!V!b3QS^QbZZlgBs!&Tgfn!&B%ps!BKppYkVQm9q@v$+%DfVlgRpL;xoHkKgOkY4$i>8Bo!F7iCb%=d61@l>wZwXC"
        "m7c`sDFDQa`B4*sQy~f=ghxK~X~Hmdo$~73E4O_M$4Fm=ldP={Tm{68z!Z{yPeHkpr?5bN3M>(dHzOheDJC#6dM*wDb`$0{i)dPY"
        "&dkgL4TWm5QIAtt?h5ixy~WMMHHV9bK?&TIV~*cq@F{#FggF+WEsOD|F+lE#ImTW_;hUIarj&CU2<8}g841MZ?8sK!X)IL4wAV5k"
        "qk(C2rCeu$X<L=s-H@izUj~IC_eX18#z_gS-3<&=X0HhgsCP)2uuNdpmgpHK-9zlUzZ%U-8JP5`)L%wO4hOp#BPPrRcCNe)lIICP"
        "$T8JW&UhLp<~GUKEMtqZ8!M|y>Tja`XJvzs6Ra6AeCWyHVq->{ggjLBQ1yH)bTx40PM==V1U228v4>}cmFQ>?j4zj<4Zg^n+Kmd3"
        "j05&rHcUSfq{z8)b^~%gJu|;%_-jQC3Kw<`3?EKh@NIC|S#6Gbu>i6Hco{GoKpX>yWAL!{>aM#1J_nOFuFh}w&@m&2&mLS-WC|^3"
        "Zy-$fv<BHq$~lXCdesE+sM9d933|LNf09v5p^z&=+y<ixV%eu`GRvvcMlmDz-UHN3FNd*=Q!7c(ydO(YG1)1LV=yi#mSRUqaOp$S"
        "j%$znMyqNqIa{nY)QYiMJ3*Ult4P4}WWB#?p$R0C%$!3R?nFP_vn`>CURR=@N6|cT5pD46u{x3Y=LhfRKE4"
    ),
    "IQ2S_GRID": ("uint64", 1024,
        "c-n=TVRqy&2!sFn3OWP#zh4`h4<lyM?!G*>+eu=Bkc4Ng^CvP&{vVN1OZI`tsPG#iqvQ|J$_M0wBIEDJ?7@*y@)v1^y)ZH=d;yX1"
        "_bywImcB0R_s4Tz<j;Ar;K=yg)i)3spJnz9X~ox#MaJjjeWO~k4M#?WCqT+XME<-oAtN!7QOdaDYofTGhxNp1>1zU?^hBnmCp0oX"
        "+wBQ{w$T&)JnlTl6Cdj&UOoA2j+eE9M8=(+R-nDwR;b9h-_i;f8F$%QAtR%ftgw-Br@s|CGVV0Dr2&A*sBl2+w48P4RwC~U0}Qp{"
        "0zi>bO9rUOxR=uawqK`{c(v34yvVpe)_@opB?qQfd<AG^loGI!KQDa+Fr}l`TnY!a<N%i(=vs2XCo}9+{m}qmp4@T)lGQgA`SR8%"
        "8{KjGBB7_=K#_4*xiwT|+}VuGUgT~gci9?m|2DF%B6+GoeKurd+^}s8y5ZOwbi*YQCXsNk#trpW+6!w9ttD&hSYZtwqtTzcdn+y@"
        "FV!BFv8W2HfJMea%EeuRpcIl5h7A3n7<67DiPcdBiY|35tJWnP$%#jqrAa_QL~=qRr~HMWBIBW%OIVTd(8(n*?j!|~@zB5}w#aze"
        "`w|^*oP-CYPdi=$WMvQ`D<t(`lA0da-yKYXJg~hxgD~0Q8)4F7a3VcSMph>$NTd-fO##7@!PPfii@U@d8BZE75tI2z$WQ>co;2JF"
        "O~R&Pt8pQ{-HDvsazX4=dJ;So#L^*r5HX1#guDp=TZc12(i8-c^(G7tzjfr%nxSSknsBgJE|9u<lg2H{PE<qk6__w&7Zo&0Rx2r*"
        "KnF}=q9dk2Jt}mb7k>)XliV&?NCHqoi|Dx3MYmkw6*kB|(sj|HQ}6&KpqRpU)aMFdqyW<4QwZtx!s2p4MB=I?mc9xkmg-F?OM~+7"
        "S!kqhjg*)!r1^>3()lDz1ht2nxov_=PhnaR`?~HMFZnishD@eVpX7JJc4rMmPy(283OdX=g*|rLUV+DoUZIx>zBXL1@E0|$W=0z`"
        "Ph)VCe13qrOB#1N;&ey%4qz4Ia38Uwd@N-QW#}k_K}F?bB)wJ2vE1a85djJE@ec7R#aT{@kXjiRkW^&g<5n3OibXL<W+ltVqLKz$"
        "Pd>(=;&V(vbyZmLv7)F>J~kBc<>Npp>oin!2y6?x%I$j@Ex8S^t<ho9Fkmt}T+&Dv$?a_!G`Wo}g9aMpcC(-=x09u1a+_G4FSmo0"
        "<K?!lT6wu$!=9B9l-sT{gfPpnSJO_FQIy-Gk}$dbDW;O!n&RwfEUAIqe$*qT;oNH9oYR{Dg(2lKUrU<CR4&i01vb#Ox^`zqCgt*2"
        "jEqOZL*V45!3BFm?xwum6M`2b4D-w7rBYtS$wkWL;NzqrX?)W6tD#15<TP2OUQTn9)=F#TG*(=)oR%gH)t2P+Ql@PhcoY%yfVGg*"
        "K#}$Gwk?ua-i`%YKqhaiN(L{Hw?|!bK#;@tV^EO8tXgRf4suvj?jC{bgM_?%Wl7~_Dd@=4U7l<X9<ZD|J+<dKkjS_5F_?fF`D=?h"
        "=D;HV^~d1CKjr`vTaiBp8JrO}VnKPp9CUc#9C*$!b4@uf`fmW*uJ*h?`ar}2mz{p!0f|;;;mkB_U=B`f2rgn{?*o;e%wbYU0HRDH"
        "=D<Z_-Ucu2EqxupnrqF3w84zTG7^yBIjE8Fw}Fj9ybW$xREh+pRy9t?RUu1h(%NwEPF)-HwwI0LNqWJTfBnMOEj0)N1So^0Fsl`k"
        "mwjDPgCg7jV8ALh;hF$KApsIfiMd*SoL)eqv;eNe%a64Sh>#qBr0KZ|Tv_BJ=XX%0L-TmHfDEMq=u+_15CFdVNZtUyx@5Kn0J1c~"
        "@?*Vf3^bnxDK5+<vbQ@Z`w22?N<*P`G*(GOZk0xR8>}OnisH{fTc_JT2JS-5vSWj4+}drfl1Y$;F2|E*VUu7R7Y~OX4)i1CFap3a"
        "F}^Jy&x#=426-k?h=Y|uAal?Mb8iFxBpRd{!kL4A+TS9gw*vr}V)ZXAul=e_LSXZt0782^FgS++m+<~OK!6A#n>d@_wAhJp9x%j7"
        "WzD!c)vVz=S5YSdNsDy=0m1UEEp%4jQs$Qs5br#wC@39fD06yJ8TUI$jvQ7$C5k*H;^uj}asLUyza4lSq{Y3mtR*FxhNv%J>x}BW"
        "UT1{K9<3v+`k1e_EiFHme|`Xg$d1G"
    ),
    "IQ3XXS_GRID": ("uint32", 256,
        "c-lpiF%Cm92tyY}Mn*<PMrQ7RtUi-3^+#6HGy!8AGqV5%+|3fKzs&%i%>0>a*1#DFbU1*ATgST?z{{=rA4H>o`wJMrGc3UZZ)VUN"
        "7kPn_2IyeDN$6rKt77hgOL4w9-<)sqf^O>^s~PUE6&R4U=Cj8*AAM049nrXANaF>*kXM`->r;^tZy{E?t)WdzR{M&NPXN#KDKM;I"
        "(ZCu+dx1e5-)4UZfk^d)k~;n*Jkcc8#7m0)msnJxcVdcxhEgY?7NGfwtm}T!pWyn?nnnaNJ>sgq{57FKXCWg%^$j{&&AvLj>}{ZB"
        "biHEjDt|?*m1ved?0wCPuYnpxk^w4>%~Kl+Bn0~e(?_FdYq3Wsu9FSp&Tg3bq(&lYCWaWf;gqXRW`G5ti$xZ*#Fd0$zyy}yHwn6+"
        "!x3+sG)0Bl=`$5hDmftJg4Ap@>@yfH9U&Y#-1cMtgral}90cLQ#)RFHquW!a98}#Cv%<(~GoVHW@X?@8{0<bn3P<d8k!HQ3ZLh<6"
        "4Uk!$p$z>R14DS7;pIjp6EnS72&@FNNm59ex>u~%h8K}!_6NkMWBC"
    ),
    "IQ3S_GRID": ("uint32", 512,
        "c-lpki;BfC2t)}YA|n3(-|iXhaw$XFH1##3eeXR34hqb>4Fe7m^mo8Ofe4<HEl^;9@o~sNvkweI3Fb4X%Rzp|4b<l(zyJ&OK;qPJ"
        "TEOR=>+1sZ1rnfvIs2}l{3Y<@84NIj4Fx=`0+(6fmjpbX10$IL4Kmp;_Q5pohO=|YhUFVzB%Q#6q?3JMUl9~xs)|mepg~X+%Oa-Y"
        "2z$-muyUC-c3GqOgmrouP?jksoO{q9g6CqtuAp{wSboK|E1wmZuh^7D=^AO7(!ssqUTzJOON8AKZLO6A=G+JSaT_AaMb>a`jx=2b"
        "1`wnra1ohq0jjuf_U4SKf@HB#>f*2sATi?OIbpPU9^RrlDv9OX3xmYMGs0+zqu8wrOc{q=fRK$@?u&bGVrqP_X7gQd0x-K3Qse|@"
        "6|BiKi6Pb%o2@#;q8K>wDa%}|N}l%sNl8?a5uvUmyiNw9-=T8_3w2(fa7D}8?B$(jtd)vM`YM6vS6EEsvab`k0BGDNuGr|>2aurW"
        "Tm$GpshceJixeRdj=niW#1-CsB%!2j7M&t+BoArHJ&jW%g%cGGL?Za4iL&s?I%=rKSFbWDoL8~7)Go5AxL?BsfuY$A&X#F0#2dR{"
        "?OHErH^SIfijh#%HvJQfx)j-llwh0DN`$5*Q7G-XhL!@whAz^jc~4+()r0%3L@2WLEa7nwpLA()KME&TjHqUdX0lXtP-i62ghF%p"
        "DyqUt^qCbc1H($ES)P#58u84shR$}7XljT6)IhbLDg+5+lRG-p_L^Lb&TYjFMvSY4N)f9eihCeQhNdvmK{6@zMBIRaCgjik_)aM`"
        "k&=;0MYu{r#5=?k3ZLYN0d8$_C)TLZNZy+QsPm$e0fs*&na#2V$Hb#)OZ3~BJC1h{VvRREW32lOs$o^Y(sZ^}x>zc;qFPRk9KJFx"
        "q`F1c6rZ;eKuv*NWW*Z|sI1sz8URXxtt=ufO&}?gMJK67uXs}ergPAvNNPTAyYb(9F(T>aM#&l(D{vIhswP%i7d7P^#Xx#!s*y~~"
        "0p;Uu@{Y&=VPdgbQ~zZ%fcUF?Lq6}<xWk@$>36e3U%!d<pdrNvhy_}Vz%|xgf0@zrZjBF(2X#RGH=Gn0D>iDvUj|AgC0{D>L;3iD"
        "(7W3;3gHjgFfq*"
    ),
    "IQ1S_GRID": ("uint32", 2048,
        "c-nQCYohI_3WO6!0FFSM{~+&I1=;KLk9&60W*H@jJPMxYc^34({ji`{e>1UWazXF=_usqT*Z+Tdix+B{CZB%vjQ$0yQUu>%`-YOO"
        "8%mZZpWJXwKCxk*FyY;sunWGip;(LgXTbx0?}Eo-?>Y!@p~F`%RPa6sbD@I>7b<ucd<&ijUIj1qE%q(;E%q(mFZM3hz;p2q-pI~="
        "3E>0q!4@)LHiE7>%q#kY&9yR~CpcI_+aqV^kQ>Uqo`47M-VLANKnVr>Sody?@Qr{Sl<*D|vLX1wo3nFx_$~PH8y)ML(AKz-o$nRj"
        "D!z00&Vm1h3f>3a2fhVeco%#NWfy$ex7dgBq?}f+6!oG+DS3^er8Fz`yjGl)E5)x-z7)tFU&5M;kTSE-#X%SF%d3(57ajBfuN0L="
        "&J54IOLL3$YeVdT2P~28LI>F{RPZ~<cA<l87b@f{_|=8rSMX!sV&CH3V((%v&zu_>*~=WGjK<a~%aq00Li^IO;AaftZHu%;%Yt9g"
        "7=#Q(hF~kln)3;E1}lTNJi~iK3IE`&eg*t<LGa&8tMxYDo=N|0{hx1&lYX&EJC<i3?b_IKK8KwbDs~?@Use`xFT9GKhaDF>@VHRH"
        "hkc8Ei+x-va)*tLqlFFm9b<k)v3d71UK!=H8Fw493|_{(#-L@aGU|4KHf$V(i%%Oke3@$lma)r8-fW}a$dSmgkt1=cK#qjAMq~+O"
        "*-#=+;7}V%<O*bBA8Z+sX+!K~j%SU?wV_0|KsNR>&xnkH^YLB$iraw#dHMbdWQG^>jL_DI%<$ozWaX}ryO8-Hb3xZ5_W>Q`y-*?V"
        "Mc#v)7h)|w$cX+fRLII6{F6IE#u6dtLB4_xG8S}2$j6>_k&8X}FyB|OIC5(4s<s2bBL}Yz1PJF~fDrG39tVZ(prHT&<JSS=a5vRK"
        "BH*{7gy+7D2R*}k!#m)cP{2Fk9q?w|yEVd}_4qfsh4+ScUi1oY_~Fm!jz9!Id>s8<<iF^R?;QAF=)n6z%;Ur81uA$S_!fLw!#fC>"
        "3!d!7kCENkpo5u$6Nhq8Q;_124sHro4rEVtFvD|r=YY2+=qZRP$UV*|1f{owpn@7w;BkeQ$%7#HA~7B(Z-Uyp<eBzLd1Kn^u00X!"
        "AZpZNuf4L6_aN(qN`J3ruKy0QUZ~)$Hy7RoUq5LVf9!*YXU#=BG^;-@2VW-mL0k?#eI1Y;WHs&%whF?}{srAHAS+n2kLT;)oSU=5"
        "D}%_gFTTim;S=yl_yl}X1fLz87hbU$H|K^Q@9`H#cy0(j%w7CSywL^no~Y+Sg}jBl#WxE61>XbD62bEz<Aqp{KOn1u{UizneT>5i"
        "V@=Xf@OOeZoRuV?M4=?ICXuX3CTkLk5<|i#4|ff(yijr1@L(R*aZdQ;;f(OwP+o}S6NmGWfY^h2;R79HyU>B>g${CE=pfgH3cdx;"
        "3(vX`{Mdt7oDtdBL+;{^k&k`MF<#kbCn+Nm!KKv+>1{}r|3E1mTcc46&c6s6YY%iGDjBjUN{1pn3}Rr3;0S9BK?FS<@xxKOGetC%"
        "5sYz!S2WLtDuO4@B+=PmN5de&9-g^+i0p#Jpyq}J-0&+15P}cfnjykK1Hl17h%M`t#lA|lPNI`YJH39X)k$~KD8JD`{H0IUbaK@%"
        "Qm2!$lB$v|iFzyDGDAv1C*f42l%rG=lU`z{(@8jez@1Rcd#A3Pl%-Uq6qS>ja?+7fQ92cc(@ai!QA$a^M+$S=Q@T@HQ%X}RQyNq1"
        "BK7IF)6iDx1pg6=A!MAetS}seN<y|mIyzNoM?ONXLc7EI>2RJ3=M%yex*fKwLpAR)eWe1WfDZM1&mo;~uaNdA1ct-k01yI_!lMDo"
        "+u_h)<oSg^=FvUw^mND^fP&5eGK3mJ1=OJ?Cd32=5;-9S*XLb_CDth%<%FXz6e$d49EC53pH%4C3ORfm1KX_Mtlbl~_%=H25T($x"
        "aYtPGF9dvUZ+FMl<=%|1TwX2|4V3IU_+!Xb44l>gCxNWb_1<<ZgQ%z7DAzw=>KTyqfhq&Bb|nKQRR!7R7mZ3nrWa#sGO-x*3Y!$)"
        "#%zpugkZAGIme7;!ZP0+vo)&9pPA;Erx97SIp&z55t&_rtB5x7ErgYA&PHG|RjyQ5s4SvuA`37g+mZSoUvVlkR9|P#6*_xxUAii*"
        "Q8v<*Z(s9V>3Ihb4k(->7}$--%v(HzOaZ;ORVH;A@X6CgHTLqSRgiP+oa6eatB;#=Onc`CQl(<4^=b7PELvTPBCQ&GE}|k4|9C*m"
        "&_vFJ{`S1!^SonZfp+PQ7Q&W!#@(A{yEo5rGs$6;{ph#)w}-JF_HGF@5!sV_KB$*_7DUb>KFwz>NRBYsY%J8bIeN+*G=PPPN!S1c"
        "9tILJ!lgtoKQIU1GRFuVJ^?0XJ$3?Xa4~y$hINS$08CBnA~f(d_y8?=Mj-eR%djN`gC}cvMjH6CM(=TX#4HiwArtY9umiyhn98$8"
        "4#9q&A<o2l)^HZiQz}Fd0)P@K2n6(>0s1Nm1oqc}{YT&(0>q?>1%dxHMZ-IV!&323T?_znh>O^i!2T2kDkxkSP!w>;kU}{Kf-*{>"
        "QicxkDWzH&Qf~SntrRI*irJ%ZDM*Km+ltzwEM0;Wwm+pIlNEPcc~PyvJr|R=l?j%QgG}J}0Heo24}~mXc%YG<5eqp=gbb`B&cdGW"
        "7IgVG>-h~!sQB*Xo74ovTf~D{%N)O@4^ZOcV&+!>xhwLNi=gR#0Aso!dfXNH6-Fw4R1l@BH7OpY=>i^CX}-KIdjGk^^}ERZUFNF`"
        "f>vKX7bgSh3w>P4aj{n@*Qgc*PZ~SKypuw=AV5YCu~G3A`qkPk^jq(j(Yp{+c2@RRLAI2|F@ne0o=lxx$SG3`5j@$&+M0rGDXXg>"
        "i|foUMDU8R>c?oIT=)qQEEj;~!cC}xjOYR{#{lKkpMmW$vdA{DJw_Jx>Nd`7kNY#Y$Tqq?hPP#S_O71+?lD4pTwELDmZu}fB}z~$"
        "z#Uzpi;FG}v*kDF6d4XOTnLS)X7qRU1{t^wPI5iNKAyE(Zy2|B!U<x=f2=jPE7~e#|691OQ!ZRppt^XyQ@~E4OX15A(H%w&z(6JK"
        "3^)dUi)~@(I1K8OW60pq-_>vQCr6P3jKjn@j2*#FhTi^h9ywc9I}vpT{)di`wcvf=Tkt*brN&@68h{S`N(9dfzXLDc@d*fC(~3RQ"
        "em&D-J=0Egk=@<Izm{yNC9A^w=@zbwa~0X|6zFS;bQRlj$Z2P~W0C4msBQVEyP-~nTb}B8*tw^RVJDAnZT=jcZ$x)G{v3W<if7u0"
        "KsdJyT{TX7@O*8>QcDqjr(2M!7S(nH8osVLRbifPC#vnHRvU=*QG2e8it}~hKdraw)?GISQkjD2zSSB^M|EcaMf>QslCp!^NNO8>"
        "?IH)0?ADNj4trSRc9649bo)uIC$*iFeVk!pf)7fPRbq{htd;MeTyFW%?P8T~yVSq!7L-@Ebok2JnZIhmOdI1&+k#^DJ=3B%(~>yM"
        "lp7h{&iFMnx(%Whh#MbjV(9JD?G4Z9Pr-33K*A{;5EUrV6MX+q%fJCsK~w>j{a3-0zzVPRmE&j1aLn5!x617^B{p+^rMb)U)8)HL"
        "ca`lb*HxmcJXcw+l3eBM0nZ;dVAem)7Ina<v{lpPnQ~T*m!%R|rEizKZn$(aM%}ki*G;9IgF2wrfjzo3bAS&8?6(8G%RnWFF7ay0"
        "ItTHbAnx+5OG5|p>~im_#0z)rT-JT1&pBP{sLbJ69S<T9=QzKTsE$gZE`#_@r0Nps@>_79rK-Y0m7N<$k18!Sl~l>?uI`?O`)(9{"
        "P+wKx>q@Vo{?jFcn@3NV1}Y1>*|c{<%7%=Bho=#dq2L+l*9j?hC#8mPPEOIVQ;<_g=7W_&Pfl#vu+a%_;G$91Ktm@dqaZ=rG+cFJ"
        "6C90(o=#dyasxG;ys{xBbLiYr9|}c!$XUWL=NM9@qPt;~GKQg3HC$4(cUIs)%qv?MYT>64GMt82f=|j6ypxB7VFq5&o^uRG<Z1FQ"
        "K@oe8Jy7t&6oM&g+Fg5;l58niqWey_N|;W%@k^(kjZUHGpL7j3r)ekU=(NmNIyq}~)+F6Y(%#Xj+zDGr*lAj+2^o~el&%PBr8I{!"
        "l<Jh;>L{(jvy=wek3!kwl=r2BGbuo!|4g_)6XO4xh|e!AxY@X-;i%N12IJEy!p%pehHOxv5UbFNzp8u9xEd4~FgzV{3AOc4m^FZi"
        "4$BI~4#R}3GocEB2~qG-S8+lSLU#D#auBo>s_Jy8Q;1V|Q%G}1QsL}$_>v2Ele1la8lZM@eDcq|%dV}ih{A-(D4p}|1~md9X~fQR"
        "n;dg((%Gh4|Cp?SjLctPCR_oSpUmC>MkX#`ROxHgHJ(8;x<VtFE5b#%Ze4YKSB=RqclG`rnS@adqxj((n1N8vr_wWOJfo^J>N%s*"
        "Po4F&`rXWx+SRyyTD8s)QYm8cNm&{MuMce5O5r1m73lKOu)@$0;DZ?F``?|1J3n9xY%Bf8F2-Ks1$tfH??=z*-~Rv~q8qC"
    ),
}

_CACHE = {}

# 7-bit sign index -> 8-bit mask: the eighth sign makes the number of negative values even.
KSIGNS = np.array([i | ((bin(i).count("1") & 1) << 7) for i in range(128)], dtype=np.uint8)


def grid(name: str) -> np.ndarray:
    """``IQ2XXS`` / ``IQ2XS`` / ``IQ2S`` -> uint8 [n, 8]; ``IQ3XXS`` / ``IQ3S`` -> uint8 [n, 4]; ``IQ1S`` -> int8 [2048, 8]."""
    if name not in _CACHE:
        dt, n, *chunks = _PACKED[name + "_GRID"]
        raw = np.frombuffer(zlib.decompress(base64.b85decode("".join(chunks))), dtype=np.dtype(dt).newbyteorder("<"))
        assert raw.size == n
        if name == "IQ1S":                      # eight nibbles per entry, each 0 / 1 / 2 for -1 / 0 / +1; values 0..3 are
            sh = np.array([0, 8, 16, 24, 4, 12, 20, 28], dtype=np.uint32)   # the low nibbles of the four bytes, 4..7 the high
            g = (((raw.astype(np.uint32)[:, None] >> sh) & 15).astype(np.int8) - 1)
        else:
            g = raw.astype(raw.dtype.newbyteorder("=")).view(np.uint8).reshape(n, -1)
        _CACHE[name] = np.ascontiguousarray(g)
    return _CACHE[name]
